// Stage 2: query-to-block scoring over a ragged batch of decode requests.
//
// score_dot: every candidate block contributes one table row (2 KiB of bf16 for 8 heads x 128)
// that is read exactly once and dotted with its request's query, so the kernel is a gather-GEMV
// bound by HBM (about 1 flop per byte); the arithmetic runs on CUDA cores, tensor cores would add
// nothing.  Rows are brought in by the copy engine (one bulk async copy per row into a per-warp
// ring in shared memory), so a warp keeps a fixed number of rows in flight without holding them
// in registers.  The grid is one resident wave (a multiple of the SM count), each warp owning a
// contiguous slice of the candidate list.  The per-KV-head query mean of the reference
// (ucm/sparse/esa/esa.py:291-296) is folded into the same kernel so that a decode step needs no
// separate prologue launch.  Under tensor parallelism the kernel also delivers its partial scores
// into every peer's inbox and raises the peers' flags when its last thread block is done: the
// all-gather half of the score all-reduce costs no launch of its own.
#include <cstdlib>

#include "common.cuh"

namespace ucmx {
namespace {

constexpr int kScoreThreads = 256;
constexpr int kMaxRingStages = 16;
constexpr int kMaxSmemOffsets = 2049;        // request offsets kept in shared memory (more requests: read from global)
constexpr int kSmemPerSm = 227 * 1024;       // shared memory of an SM that thread blocks can have
constexpr int kRingStages = 4;               // rows of 2 KiB and more a warp keeps in flight: two pairs (measured: six are 7 % slower)

// ------------------------------------------------------------------ query group mean

__global__ void query_group_mean_kernel(const uint16_t* __restrict__ q, int n_tok, int Hq, int Hkv, int D,
                                        int64_t tok_stride, int round_bf16, float* __restrict__ out)
{
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per_tok = (int64_t)Hkv * D;
    if (idx >= (int64_t)n_tok * per_tok) return;
    const int t = (int)(idx / per_tok);
    const int rem = (int)(idx - (int64_t)t * per_tok);
    const int h = rem / D, d = rem - h * D;
    const uint16_t* qt = q + (int64_t)t * tok_stride;
    float v;
    if (Hq >= Hkv) {
        const int g = Hq / Hkv;
        float acc = __uint_as_float((uint32_t)qt[(int64_t)(h * g) * D + d] << 16);
        for (int j = 1; j < g; ++j) acc += __uint_as_float((uint32_t)qt[(int64_t)(h * g + j) * D + d] << 16);
        acc *= 1.0f / (float)g;
        v = round_bf16 ? bf16_round(acc) : acc;
    } else {
        const int r = Hkv / Hq;
        v = __uint_as_float((uint32_t)qt[(int64_t)(h / r) * D + d] << 16);
    }
    out[idx] = v;
}

// ------------------------------------------------------------------ fast path: n_rep == 1

struct ScoreParams {
    const void* reps;
    int64_t n_slots;         // rows of the table; a slot id at or beyond it is skipped and reported
    const int32_t* offsets;
    const int32_t* slot_ids;
    const float* q;          // fp32 [n_req, E] (already reduced per KV head), or NULL
    const uint16_t* q_raw;   // bf16 [n_req, Hq, D] when the group mean is folded in
    int64_t q_raw_stride;    // elements between requests in q_raw
    int32_t Hq, D, round_bf16;
    float* out;              // may be NULL when the scores only go to the peers' inboxes
    int32_t n_req, total, E;
    float scale;
    int32_t stages;          // ring depth per warp
    int32_t rows_per_warp;   // candidates per warp (the last warps may get fewer or none)
    int32_t d_shift;         // log2(D) when D is a power of two, else -1
    PeerPush px;             // px.world == 0: single rank
    int32_t* err;
    int32_t early;           // launched so that it may begin before the kernel ahead of it in the stream has ended
};

// N partial sums per lane, each to be added up over the 16 lanes of a half-warp: instead of N butterflies of four
// steps, the lanes first split the values between them - at distance 1 the even lanes keep the lower half of the
// values and the odd lanes the upper half, each adding what its neighbour sends, and so on with half as many values
// at twice the distance - and the steps that are left finish the one value a lane still holds.  The lane ends up
// with the total of value number (bit 0 of the lane, bit 1, ...) read as a binary number from the top:
// N - 1 + (4 - log2 N) shuffles instead of 4 N.
template <int N, int DIST>
__device__ __forceinline__ float half_warp_sums(float (&v)[N], int lane)
{
    if constexpr (N == 1) {
        float x = v[0];
#pragma unroll
        for (int o = DIST; o < 16; o <<= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        return x;
    } else {
        static_assert(DIST < 16, "at most sixteen values");
        float w[N / 2];
        const bool upper = (lane & DIST) != 0;
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            const float keep = upper ? v[i + N / 2] : v[i];
            const float send = upper ? v[i] : v[i + N / 2];
            w[i] = keep + __shfl_xor_sync(0xffffffffu, send, DIST);
        }
        return half_warp_sums<N / 2, DIST * 2>(w, lane);
    }
}

// eight products of fp32 q with a 16-byte piece of bf16 values, as four packed multiply-adds
__device__ __forceinline__ float dot8_packed(const float4& q0, const float4& q1, const uint4& x)
{
    float2 s0 = __fmul2_rn(make_float2(q0.x, q0.y), make_float2(bf16lo(x.x), bf16hi(x.x)));
    float2 s1 = __fmul2_rn(make_float2(q0.z, q0.w), make_float2(bf16lo(x.y), bf16hi(x.y)));
    s0 = __ffma2_rn(make_float2(q1.x, q1.y), make_float2(bf16lo(x.z), bf16hi(x.z)), s0);
    s1 = __ffma2_rn(make_float2(q1.z, q1.w), make_float2(bf16lo(x.w), bf16hi(x.w)), s1);
    return (s0.x + s1.x) + (s0.y + s1.y);
}

// Element layout per lane: a row is cut into 16-byte pieces; piece j of a row belongs to lane
// j % 32.  A piece holds 8 bf16 or 4 fp32 values.  QN = E/32 values of q per lane.
// With R >= 2 representatives per head (bf16, 128 channels per head: GSA's tables) a 128-channel vector is 16 pieces,
// so lanes 0-15 hold one vector of piece i and lanes 16-31 the next: the two (of R) representatives i * 2 and
// i * 2 + 1 of head i / (R / 2).  The score is then the sum over heads of the best representative's dot product.
template <int DT, int QN, int R = 1>
struct RowDot {
    static constexpr int kPerPiece = (DT == UCMX_DT_BF16) ? 8 : 4;
    static constexpr int kPieces = QN / kPerPiece;
    static constexpr int kLoadsPerHead = R >= 2 ? R / 2 : 1;
    static constexpr int kHeads = kPieces / kLoadsPerHead;       // (R >= 2)

    float q[QN];

    // R >= 2: this lane's eight channels of every head's query; qrow is fp32 [kHeads][128]
    __device__ __forceinline__ void load_q_reps(const float* __restrict__ qrow, int lane)
    {
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            const float4* src = reinterpret_cast<const float4*>(qrow + h * 128 + (lane & 15) * 8);
            const float4 f0 = __ldg(src), f1 = __ldg(src + 1);
            q[h * 8 + 0] = f0.x;
            q[h * 8 + 1] = f0.y;
            q[h * 8 + 2] = f0.z;
            q[h * 8 + 3] = f0.w;
            q[h * 8 + 4] = f1.x;
            q[h * 8 + 5] = f1.y;
            q[h * 8 + 6] = f1.z;
            q[h * 8 + 7] = f1.w;
        }
    }
    // R >= 2: every piece's dot product with its head's query (this lane's eight channels) ...
    __device__ __forceinline__ void partial_reps(const uint4 (&buf)[kPieces], float (&part)[kPieces]) const
    {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const int h = i / kLoadsPerHead;
            part[i] = dot8_packed(make_float4(q[h * 8 + 0], q[h * 8 + 1], q[h * 8 + 2], q[h * 8 + 3]),
                                  make_float4(q[h * 8 + 4], q[h * 8 + 5], q[h * 8 + 6], q[h * 8 + 7]), buf[i]);
        }
    }
    // ... and the score in every lane: all pieces summed over the half-warps at once (piece i = h * kLoadsPerHead + j
    // ends up in the lane whose low bits, most significant first, spell i), the maximum over a head's pieces (lanes
    // kHeads and more apart) and over the two half-warps, the sum over the heads (the lane bits below)
    __device__ __forceinline__ float reduce_reps(float (&part)[kPieces], int lane) const
    {
        float t = half_warp_sums<kPieces, 1>(part, lane);
#pragma unroll
        for (int o = kHeads; o < kPieces; o <<= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 16));
#pragma unroll
        for (int o = 1; o < kHeads; o <<= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        return t;
    }

    __device__ __forceinline__ void load_q(const float* __restrict__ qrow, int lane)
    {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const float4* src = reinterpret_cast<const float4*>(qrow + (i * 32 + lane) * kPerPiece);
#pragma unroll
            for (int v = 0; v < kPerPiece / 4; ++v) {
                const float4 f = __ldg(src + v);
                q[i * kPerPiece + v * 4 + 0] = f.x;
                q[i * kPerPiece + v * 4 + 1] = f.y;
                q[i * kPerPiece + v * 4 + 2] = f.z;
                q[i * kPerPiece + v * 4 + 3] = f.w;
            }
        }
    }
    __device__ __forceinline__ void load_q_smem(const float* qrow, int lane)
    {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const float4* src = reinterpret_cast<const float4*>(qrow + (i * 32 + lane) * kPerPiece);
#pragma unroll
            for (int v = 0; v < kPerPiece / 4; ++v) {
                const float4 f = src[v];
                q[i * kPerPiece + v * 4 + 0] = f.x;
                q[i * kPerPiece + v * 4 + 1] = f.y;
                q[i * kPerPiece + v * 4 + 2] = f.z;
                q[i * kPerPiece + v * 4 + 3] = f.w;
            }
        }
    }
    // q from the raw bf16 query [Hq, D]: mean over the head group in fp32 (heads in ascending order, times 1/group),
    // optionally rounded to bf16 - the arithmetic of query_group_mean_kernel.  This is the warp's own route for a
    // request the thread block has not staged (a slice that touches more than a few requests); it is kept small
    // rather than fast: rolled loops, one head at a time.
    __device__ __forceinline__ void load_q_raw(const uint16_t* __restrict__ qreq, int lane, int Hq, int Hkv, int D,
                                               int round_bf16)
    {
        const int g = Hq >= Hkv ? Hq / Hkv : 1;
        const int rep = Hq >= Hkv ? 1 : Hkv / Hq;
        const float inv = Hq >= Hkv ? 1.0f / (float)g : 1.0f;
        const bool rnd = Hq >= Hkv && round_bf16;
#pragma unroll 1
        for (int c = 0; c < QN / 4; ++c) {
            const int i = c / (kPerPiece / 4), half = c % (kPerPiece / 4);
            const int e0 = (i * 32 + lane) * kPerPiece + half * 4;
            const int h = e0 / D, d = e0 - h * D;
            const uint16_t* src = qreq + (int64_t)((h / rep) * g) * D + d;
            uint2 w = __ldg(reinterpret_cast<const uint2*>(src));
            float a0 = bf16lo(w.x), a1 = bf16hi(w.x), a2 = bf16lo(w.y), a3 = bf16hi(w.y);
#pragma unroll 1
            for (int j = 1; j < g; ++j) {
                w = __ldg(reinterpret_cast<const uint2*>(src + (int64_t)j * D));
                a0 += bf16lo(w.x);
                a1 += bf16hi(w.x);
                a2 += bf16lo(w.y);
                a3 += bf16hi(w.y);
            }
            a0 *= inv;
            a1 *= inv;
            a2 *= inv;
            a3 *= inv;
            if (rnd) {
                a0 = bf16_round(a0);
                a1 = bf16_round(a1);
                a2 = bf16_round(a2);
                a3 = bf16_round(a3);
            }
            set_q4(c, a0, a1, a2, a3);
        }
    }
    // q[4c .. 4c+3] = values, c known only at run time (a chain of selects: the array must stay in registers)
    __device__ __forceinline__ void set_q4(int c, float a0, float a1, float a2, float a3)
    {
#pragma unroll
        for (int k = 0; k < QN / 4; ++k)
            if (k == c) {
                q[k * 4 + 0] = a0;
                q[k * 4 + 1] = a1;
                q[k * 4 + 2] = a2;
                q[k * 4 + 3] = a3;
            }
    }
    __device__ __forceinline__ void load_row(const void* row, int lane, uint4 (&buf)[kPieces]) const
    {
        const uint4* src = reinterpret_cast<const uint4*>(row);
#pragma unroll
        for (int i = 0; i < kPieces; ++i) buf[i] = ld_stream16(src + i * 32 + lane);
    }
    __device__ __forceinline__ void zero_row(uint4 (&buf)[kPieces]) const
    {
#pragma unroll
        for (int i = 0; i < kPieces; ++i) buf[i] = make_uint4(0, 0, 0, 0);
    }
    // The lane's share of q . row.  bf16 rows go through the packed fp32 multiply-add (two products per instruction)
    // into two independent pairs of partial sums: half the instructions of a scalar chain and a quarter of its depth.
    __device__ __forceinline__ float dot(const uint4 (&buf)[kPieces]) const
    {
        if (DT == UCMX_DT_BF16) {
            float2 s0 = make_float2(0.0f, 0.0f), s1 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < kPieces; ++i) {
                const uint4 v = buf[i];
                s0 = __ffma2_rn(make_float2(q[i * 8 + 0], q[i * 8 + 1]), make_float2(bf16lo(v.x), bf16hi(v.x)), s0);
                s1 = __ffma2_rn(make_float2(q[i * 8 + 2], q[i * 8 + 3]), make_float2(bf16lo(v.y), bf16hi(v.y)), s1);
                s0 = __ffma2_rn(make_float2(q[i * 8 + 4], q[i * 8 + 5]), make_float2(bf16lo(v.z), bf16hi(v.z)), s0);
                s1 = __ffma2_rn(make_float2(q[i * 8 + 6], q[i * 8 + 7]), make_float2(bf16lo(v.w), bf16hi(v.w)), s1);
            }
            return (s0.x + s1.x) + (s0.y + s1.y);
        }
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const uint4 v = buf[i];
            if (DT == UCMX_DT_BF16) {
                acc = fmaf(q[i * 8 + 0], bf16lo(v.x), acc);
                acc = fmaf(q[i * 8 + 1], bf16hi(v.x), acc);
                acc = fmaf(q[i * 8 + 2], bf16lo(v.y), acc);
                acc = fmaf(q[i * 8 + 3], bf16hi(v.y), acc);
                acc = fmaf(q[i * 8 + 4], bf16lo(v.z), acc);
                acc = fmaf(q[i * 8 + 5], bf16hi(v.z), acc);
                acc = fmaf(q[i * 8 + 6], bf16lo(v.w), acc);
                acc = fmaf(q[i * 8 + 7], bf16hi(v.w), acc);
            } else {
                acc = fmaf(q[i * 4 + 0], __uint_as_float(v.x), acc);
                acc = fmaf(q[i * 4 + 1], __uint_as_float(v.y), acc);
                acc = fmaf(q[i * 4 + 2], __uint_as_float(v.z), acc);
                acc = fmaf(q[i * 4 + 3], __uint_as_float(v.w), acc);
            }
        }
        return acc;
    }
};

// One warp per table row, rows fetched by the copy engine: every warp owns a contiguous slice of the
// candidate list and a private ring of `stages` row buffers in shared memory.  Lane 0 keeps the ring full with
// one bulk async copy per row (completion on the stage's mbarrier); the warp takes rows out of shared memory
// two at a time (two independent multiply-add chains and one interleaved reduction), and the stages are
// refilled before the partial sums are even added up, so a warp has `stages` rows in flight at all times
// without holding any of them in registers.  Scores are collected one per lane and leave 32 at a time.  With a
// peer exchange (tensor-parallel ranks) every score is also written into each rank's inbox, so the exchange of
// partial scores rides on the scoring kernel's own stores.
// The kernel is as much bound by instruction issue as by memory (a row of 2 KiB is 130 instructions of a warp
// against 50 ns of HBM time per SM), so everything outside the row loop is kept short: no 64-bit divisions, the
// stage index counted instead of computed, slot ids read once.
// PEER: the scores also go to the ranks' inboxes (tensor-parallel retrieval).  A template switch rather than a test of
// p.px.world: the exchange's stores and round counters are inlined wherever scores leave, a fifth of the kernel's
// instruction stream, and a single rank's launches - short kernels that start with cold instruction caches - should
// not carry them.
template <int DT, int QN, bool FUSEQ, int R = 1, bool PEER = false>
__global__ void __launch_bounds__(kScoreThreads, 2) score_dot_ring_kernel(ScoreParams p)
{
    static_assert(R == 1 || (!FUSEQ && DT == UCMX_DT_BF16), "several representatives per head: bf16 tables, fp32 queries");
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kWarps = kScoreThreads / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int w = (int)blockIdx.x * kWarps + warp;
    const int begin = min(w * p.rows_per_warp, p.total);
    const int end = min(begin + p.rows_per_warp, p.total);
    // An early launch reads its inputs (offsets, slot ids, table rows, queries: none of them written by the kernel
    // ahead) while that kernel's last thread blocks are still running, and waits for its end only before its own
    // first store.  The kernel behind this one is let in right away, whichever it is: another scoring launch on the
    // same terms, or the top-k, which is always launched that way and waits for this kernel's end before it reads.
    early_start_allow();

    using RD = RowDot<DT, QN, R>;
    constexpr uint32_t kRowBytes = (uint32_t)QN * 32u * (DT == UCMX_DT_BF16 ? 2u : 4u);
    constexpr int E = QN * 32 / R;            // elements of a query row
    const int stages = p.stages;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem) + warp * kMaxRingStages;
    unsigned char* ring = smem + (size_t)kWarps * kMaxRingStages * 8 + (size_t)warp * stages * kRowBytes;
    const unsigned char* base = reinterpret_cast<const unsigned char*>(p.reps);

    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
    }
    __syncwarp();

    uint32_t round = 0;
    int64_t push_off = 0;
    if (PEER) {
        round = peer_round_now(p.px);
        push_off = peer_inbox_offset(p.px, round, p.px.my_rank);
    }
    // A decode step runs this kernel right after gigabytes of block traffic, so nothing it needs is in L2.  What
    // does not depend on anything is therefore requested first and used late: the request offsets (one coalesced
    // read per thread block, searched in shared memory afterwards) and the slot ids; the rows follow as soon as
    // the slot ids are there, and the query while the rows are on their way.
    // (the offsets sit behind the rings in dynamic shared memory, sized for this batch: a fixed array for the largest
    // batch would cost every launch 8 KiB that the rings can use)
    int32_t* s_off = reinterpret_cast<int32_t*>(smem + (size_t)kWarps * kMaxRingStages * 8 + (size_t)kWarps * stages * kRowBytes);
    const bool off_in_smem = p.n_req + 1 <= kMaxSmemOffsets;
    constexpr int kOffIters = (kMaxSmemOffsets + kScoreThreads - 1) / kScoreThreads;
    int32_t off_reg[kOffIters];
    if (off_in_smem) {
#pragma unroll
        for (int j = 0; j < kOffIters; ++j) {
            const int i = (int)threadIdx.x + j * kScoreThreads;
            off_reg[j] = i <= p.n_req ? __ldg(p.offsets + i) : 0;
        }
    }
    const uint64_t read_once = l2_evict_first_policy();      // every table row is read exactly once

    // slot id of a row; one outside the table is reported and treated as empty
    auto slot_of = [&](int row) -> int {
        if (row >= end) return -1;
        int v = p.slot_ids ? __ldg(p.slot_ids + row) : row;
        if (v >= 0 && (int64_t)v >= p.n_slots) {
            if (p.err) atomicExch(p.err, 3);
            v = -1;
        }
        return v;
    };
    uint32_t valid = 0;        // bit s: stage s holds (or is about to hold) a row
    auto fetch = [&](int s, int slot) {
        if (slot >= 0) {
            valid |= 1u << s;
            if (lane == 0) {
                mbar_expect_tx(&full[s], kRowBytes);
                bulk_g2s_hint(ring + (size_t)s * kRowBytes, base + (size_t)slot * kRowBytes, kRowBytes, &full[s], read_once);
            }
        } else {
            valid &= ~(1u << s);
        }
    };
    // Slot ids come 32 at a time, one per lane with one coalesced read, a batch ahead of the rows that need them (a
    // warp of the decode batch has about fifteen rows: one read), and are handed round by shuffles: no row waits for
    // a trip to memory for its id.
    int ids_base = begin;                                    // ids_cur: rows [ids_base, ids_base + 32), ids_nxt: the 32 after
    int ids_cur = slot_of(begin + lane), ids_nxt = slot_of(begin + 32 + lane);
    auto slot_at = [&](int row) -> int {                     // (called by the whole warp, rows in ascending order)
        if (row - ids_base >= 32) {                          // into the next batch: the one after it is asked for now
            ids_base += 32;
            ids_cur = ids_nxt;
            ids_nxt = slot_of(ids_base + 32 + lane);
        }
        return __shfl_sync(0xffffffffu, ids_cur, (row - ids_base) & 31);
    };
    if (begin < end) {
        for (int s = 0; s < stages; ++s) fetch(s, slot_at(begin + s));
    }
    if (off_in_smem) {
#pragma unroll
        for (int j = 0; j < kOffIters; ++j) {
            const int i = (int)threadIdx.x + j * kScoreThreads;
            if (i <= p.n_req) s_off[i] = off_reg[j];
        }
    }
    __syncthreads();
    const int32_t* off = off_in_smem ? s_off : p.offsets;
    const int Hkv = E / p.D;

    // With the query mean folded in, the thread block reduces the raw queries of the (at most kStagedReq) requests
    // its slice touches first into shared memory, all threads at once and every load requested before the first
    // sum; a warp that runs past them reduces its query on its own.
    constexpr int kStagedReq = 3;
    __shared__ __align__(16) float s_q[FUSEQ ? kStagedReq * E : 4];
    int r_cta = 0;
    if (FUSEQ) {
        const int cta_begin = min((int)blockIdx.x * kWarps * p.rows_per_warp, p.total);
        {
            int lo = 0, hi = p.n_req;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (off[mid] <= cta_begin) lo = mid; else hi = mid;
            }
            r_cta = lo;
        }
        const int g = p.Hq >= Hkv ? p.Hq / Hkv : 1;
        const int rep = p.Hq >= Hkv ? 1 : Hkv / p.Hq;
        const float inv = 1.0f / (float)g;
        constexpr int kIters = (kStagedReq * (E / 4) + kScoreThreads - 1) / kScoreThreads;   // chunks of 4 elements per thread
        uint2 w4[kIters][4];
        const uint16_t* srcs[kIters];
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
            const int idx = (int)threadIdx.x + it * kScoreThreads;
            const int rr = idx / (E / 4);
            const int e0 = (idx - rr * (E / 4)) * 4;
            const int req = r_cta + rr;
            srcs[it] = nullptr;
            if (rr < kStagedReq && req < p.n_req) {
                const int h = p.d_shift >= 0 ? (e0 >> p.d_shift) : e0 / p.D;
                const int d = e0 - h * p.D;
                srcs[it] = p.q_raw + (int64_t)req * p.q_raw_stride + (int64_t)((h / rep) * g) * p.D + d;
                if (g == 4) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) w4[it][j] = __ldg(reinterpret_cast<const uint2*>(srcs[it] + (int64_t)j * p.D));
                }
            }
        }
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
            if (!srcs[it]) continue;
            const int idx = (int)threadIdx.x + it * kScoreThreads;
            float a0, a1, a2, a3;
            if (g == 4) {
                a0 = ((bf16lo(w4[it][0].x) + bf16lo(w4[it][1].x)) + bf16lo(w4[it][2].x)) + bf16lo(w4[it][3].x);
                a1 = ((bf16hi(w4[it][0].x) + bf16hi(w4[it][1].x)) + bf16hi(w4[it][2].x)) + bf16hi(w4[it][3].x);
                a2 = ((bf16lo(w4[it][0].y) + bf16lo(w4[it][1].y)) + bf16lo(w4[it][2].y)) + bf16lo(w4[it][3].y);
                a3 = ((bf16hi(w4[it][0].y) + bf16hi(w4[it][1].y)) + bf16hi(w4[it][2].y)) + bf16hi(w4[it][3].y);
            } else {
                uint2 w0 = __ldg(reinterpret_cast<const uint2*>(srcs[it]));
                a0 = bf16lo(w0.x), a1 = bf16hi(w0.x), a2 = bf16lo(w0.y), a3 = bf16hi(w0.y);
                for (int j = 1; j < g; ++j) {
                    const uint2 wj = __ldg(reinterpret_cast<const uint2*>(srcs[it] + (int64_t)j * p.D));
                    a0 += bf16lo(wj.x);
                    a1 += bf16hi(wj.x);
                    a2 += bf16lo(wj.y);
                    a3 += bf16hi(wj.y);
                }
            }
            if (p.Hq >= Hkv) {
                a0 *= inv;
                a1 *= inv;
                a2 *= inv;
                a3 *= inv;
                if (p.round_bf16) {
                    a0 = bf16_round(a0);
                    a1 = bf16_round(a1);
                    a2 = bf16_round(a2);
                    a3 = bf16_round(a3);
                }
            }
            *reinterpret_cast<float4*>(&s_q[idx * 4]) = make_float4(a0, a1, a2, a3);
        }
        __syncthreads();
    }

    if (begin < end) {
        RD rd;
        int r;
        {
            int lo = 0, hi = p.n_req;             // invariant: off[lo] <= begin < off[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (off[mid] <= begin) lo = mid; else hi = mid;
            }
            r = lo;
        }
        int r_end = off[r + 1];
        auto fetch_q = [&](int req) {
            if (FUSEQ) {
                if (req >= r_cta && req < r_cta + kStagedReq) rd.load_q_smem(&s_q[(req - r_cta) * E], lane);
                else rd.load_q_raw(p.q_raw + (int64_t)req * p.q_raw_stride, lane, p.Hq, Hkv, p.D, p.round_bf16);
            } else if (R > 1) {
                rd.load_q_reps(p.q + (int64_t)req * E, lane);
            } else {
                rd.load_q(p.q + (int64_t)req * E, lane);
            }
        };
        fetch_q(r);

        float mine = 0.0f;        // score of row (flush_from + lane), once computed
        int flush_from = begin;
        uint32_t phase = 0;       // bit s: parity of the next completion of stage s
        bool failed = false;
        auto flush = [&](int upto) {   // rows [flush_from, upto), upto - flush_from <= 32
            const int row = flush_from + lane;
            if (p.early) early_start_wait();
            if (row < upto) {
                if (p.out) p.out[row] = mine;
                if (PEER) {
                    for (int t = 0; t < p.px.world; ++t)
                        reinterpret_cast<float*>(p.px.bases[t] + push_off)[row] = mine;
                }
            }
            flush_from = upto;
        };
        // the row in stage s as 16-byte pieces (zeros when the stage holds nothing or its copy never landed)
        auto take = [&](int s, uint4 (&buf)[RD::kPieces]) -> bool {
            const bool has = (valid >> s) & 1u;
            bool ok = has && !failed;
            if (ok && !mbar_wait(&full[s], (phase >> s) & 1u)) {
                failed = true;                          // the copy never landed: report, stop fetching
                if (p.err) atomicExch(p.err, 1);
                ok = false;
            }
            if (ok) {
                phase ^= 1u << s;
                const uint4* src = reinterpret_cast<const uint4*>(ring + (size_t)s * kRowBytes);
#pragma unroll
                for (int i = 0; i < RD::kPieces; ++i) buf[i] = src[i * 32 + lane];
            } else {
                rd.zero_row(buf);
            }
            return has;
        };
        auto keep = [&](int row, bool has, float v) {
            if (lane == ((row - flush_from) & 31)) mine = has ? v * p.scale : -INFINITY;
            if (row - flush_from == 31) flush(row + 1);
        };

        int cs = 0;               // stage of the row being consumed (rows take the stages round robin)
        int row = begin;
        while (row < end) {
            if (row >= r_end) {
                do {
                    ++r;
                    r_end = off[r + 1];
                } while (row >= r_end);
                fetch_q(r);
            }
            const int cs1 = cs + 1 == stages ? 0 : cs + 1;
            if (R == 1 && QN <= 32 && row + 1 < end && row + 1 < r_end) {        // (the widest rows leave no registers for a pair)
                // two rows of one request: independent chains, one interleaved reduction
                const int n0 = slot_at(row + stages), n1 = slot_at(row + 1 + stages);
                uint4 a[RD::kPieces], b[RD::kPieces];
                const bool ha = take(cs, a);
                const bool hb = take(cs1, b);
                float x = rd.dot(a), y = rd.dot(b);
                __syncwarp();                           // every lane has taken its part of both stages
                if (!failed) {
                    fetch(cs, n0);
                    fetch(cs1, n1);
                }
                // One reduction for both rows: neighbouring lanes first swap what the other one sums, so that the lanes
                // whose parity is that of the first row's place in the output batch add up the first row and the others
                // the second; four more steps and every lane holds the total its parity stands for - among them the two
                // lanes that keep these rows' scores.
                {
                    const bool second = (lane ^ (row - flush_from)) & 1;
                    const float got = __shfl_xor_sync(0xffffffffu, second ? x : y, 1);
                    float z = (second ? y : x) + got;
#pragma unroll
                    for (int o = 2; o < 32; o <<= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
                    x = y = z;
                }
                keep(row, ha, x);
                keep(row + 1, hb, y);
                row += 2;
                cs = cs1 + 1 == stages ? 0 : cs1 + 1;
            } else {
                const int n0 = slot_at(row + stages);
                uint4 a[RD::kPieces];
                const bool ha = take(cs, a);
                float x;
                if constexpr (R == 1) {
                    x = rd.dot(a);
                    __syncwarp();
                    if (!failed) fetch(cs, n0);
                    x = warp_sum(x);
                } else {
                    float part[RD::kPieces];
                    rd.partial_reps(a, part);
                    __syncwarp();
                    if (!failed) fetch(cs, n0);
                    x = rd.reduce_reps(part, lane);
                }
                keep(row, ha, x);
                row += 1;
                cs = cs1;
            }
        }
        flush(end);
    }
    if (PEER) peer_publish_round(p.px, round);
}

// ------------------------------------------------------------------ general path: any n_rep

struct ScoreGenParams {
    const void* reps;
    int64_t n_slots;
    const int32_t* offsets;
    const int32_t* slot_ids;
    const float* q;
    float* out;
    int32_t n_req, total, H, R, D;
    float scale;
    PeerPush px;
    int32_t* err;
};

// slot id of candidate c, or -1 for an empty entry; an id beyond the table is reported (code 3) and skipped
__device__ __forceinline__ int checked_slot(const int32_t* __restrict__ slot_ids, int64_t c, int64_t n_slots, int32_t* err)
{
    const int slot = slot_ids ? __ldg(slot_ids + c) : (int)c;
    if (slot >= 0 && (int64_t)slot >= n_slots) {
        if (err) atomicExch(err, 3);
        return -1;
    }
    return slot;
}

// One warp per candidate.  For each KV head the warp takes the dot product of the query head with
// each of the block's n_rep representatives and keeps the largest; head results are summed
// (TopkBlockSelector::ComputeBlockScore, ucm/sparse/gsa/offload_ops/src/select_topk_block.cpp:53-76).
template <int DT>
__global__ void __launch_bounds__(kScoreThreads) score_dot_general_kernel(ScoreGenParams p)
{
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    constexpr int kPer = (DT == UCMX_DT_BF16) ? 8 : 4;
    const int pieces = p.D / kPer;
    const size_t esz = (DT == UCMX_DT_BF16) ? 2 : 4;
    const size_t row_elems = (size_t)p.H * p.R * p.D;
    const unsigned char* base = reinterpret_cast<const unsigned char*>(p.reps);

    for (int64_t c = w0; c < p.total; c += W) {
        const int r = find_request(p.offsets, p.n_req, (int)c);
        const int slot = checked_slot(p.slot_ids, c, p.n_slots, p.err);
        if (slot < 0) {
            if (lane == 0) p.out[c] = -INFINITY;
            continue;
        }
        const float* qr = p.q + (int64_t)r * p.H * p.D;
        const unsigned char* row = base + (size_t)slot * row_elems * esz;
        float total = 0.0f;
        for (int h = 0; h < p.H; ++h) {
            float best = -INFINITY;
            for (int j = 0; j < p.R; ++j) {
                const unsigned char* kv = row + ((size_t)h * p.R + j) * p.D * esz;
                float acc = 0.0f;
                for (int pc = lane; pc < pieces; pc += 32) {
                    const uint4 v = ld_stream16(kv + (size_t)pc * 16);
                    const float* qq = qr + h * p.D + pc * kPer;
                    if (DT == UCMX_DT_BF16) {
                        acc = fmaf(__ldg(qq + 0), bf16lo(v.x), acc);
                        acc = fmaf(__ldg(qq + 1), bf16hi(v.x), acc);
                        acc = fmaf(__ldg(qq + 2), bf16lo(v.y), acc);
                        acc = fmaf(__ldg(qq + 3), bf16hi(v.y), acc);
                        acc = fmaf(__ldg(qq + 4), bf16lo(v.z), acc);
                        acc = fmaf(__ldg(qq + 5), bf16hi(v.z), acc);
                        acc = fmaf(__ldg(qq + 6), bf16lo(v.w), acc);
                        acc = fmaf(__ldg(qq + 7), bf16hi(v.w), acc);
                    } else {
                        acc = fmaf(__ldg(qq + 0), __uint_as_float(v.x), acc);
                        acc = fmaf(__ldg(qq + 1), __uint_as_float(v.y), acc);
                        acc = fmaf(__ldg(qq + 2), __uint_as_float(v.z), acc);
                        acc = fmaf(__ldg(qq + 3), __uint_as_float(v.w), acc);
                    }
                }
                acc = warp_sum(acc);
                best = fmaxf(best, acc);
            }
            total += best;
        }
        if (lane == 0) p.out[c] = total * p.scale;
    }
}

// The same for the shape GSA uses - bf16, 128 channels per head, a power-of-two number of representatives - with
// the whole row in flight at once: a vector of 128 bf16 is 16 lanes of 16 bytes, so a warp-wide load brings two
// vectors (for two representatives per head: both representatives of one head), NV = H * n_rep / 2 loads bring the
// row, and all of them are requested before the first is used.  Each half-warp reduces its vector's dot product
// (four shuffle steps); the best of a head's representatives is a maximum over the head's loads and, last, over
// the two halves.  Slot ids are read a candidate ahead.
template <int NV, int R>
__global__ void __launch_bounds__(kScoreThreads) score_dot_reps_kernel(ScoreGenParams p)
{
    static_assert(R >= 2 && (R & (R - 1)) == 0, "representatives per head: a power of two, at least 2");
    constexpr int kLoadsPerHead = R / 2;
    constexpr int kHeads = NV / kLoadsPerHead;
    const int lane = threadIdx.x & 31, half = lane >> 4, pc = lane & 15;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int begin = (int)((int64_t)p.total * w / W);
    const int end = (int)((int64_t)p.total * (w + 1) / W);
    if (begin >= end) return;
    const unsigned char* base = reinterpret_cast<const unsigned char*>(p.reps);
    constexpr size_t kRowBytes = (size_t)NV * 512;
    int slot_next = checked_slot(p.slot_ids, begin, p.n_slots, p.err);
    int r = find_request(p.offsets, p.n_req, begin);
    int r_end = __ldg(p.offsets + r + 1);
    for (int c = begin; c < end; ++c) {
        const int slot = slot_next;
        if (c + 1 < end) slot_next = checked_slot(p.slot_ids, c + 1, p.n_slots, p.err);
        if (slot < 0) {
            if (lane == 0) p.out[c] = -INFINITY;
            continue;
        }
        uint4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = ld_stream16(base + (size_t)slot * kRowBytes + (size_t)i * 512 + (size_t)lane * 16);
        while (c >= r_end) {
            ++r;
            r_end = __ldg(p.offsets + r + 1);
        }
        const float* qr = p.q + (int64_t)r * kHeads * 128 + pc * 8;
        // every load's dot product with its head's query (this lane's eight channels), then all NV of them summed
        // over the half-warp at once: the lane is left with the product of load number sel(lane)
        float part[NV];
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            const float4 q0 = __ldg(reinterpret_cast<const float4*>(qr + h * 128));
            const float4 q1 = __ldg(reinterpret_cast<const float4*>(qr + h * 128) + 1);
#pragma unroll
            for (int j = 0; j < kLoadsPerHead; ++j) part[h * kLoadsPerHead + j] = dot8_packed(q0, q1, v[h * kLoadsPerHead + j]);
        }
        float total = half_warp_sums<NV, 1>(part, lane);
        // load i = h * kLoadsPerHead + j sits in the lane whose low bits, most significant first, spell i: the loads of
        // one head differ in the lane bits from kHeads upwards, the heads in the bits below
#pragma unroll
        for (int o = kHeads; o < NV; o <<= 1) total = fmaxf(total, __shfl_xor_sync(0xffffffffu, total, o));
        total = fmaxf(total, __shfl_xor_sync(0xffffffffu, total, 16));        // the other half-warp's representatives
#pragma unroll
        for (int o = 1; o < kHeads; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) p.out[c] = total * p.scale;
        (void)half;
    }
}

// Launch geometry of the ring kernel: one resident wave of `ctas_per_sm` thread blocks of 8 warps per SM, the
// shared memory of an SM split evenly between the warps' rings.
struct RingGeometry {
    int grid, stages;
    size_t smem;
};

RingGeometry ring_geometry(int32_t total, uint32_t row_bytes, int32_t n_req, size_t static_bytes)
{
    constexpr int warps_per_cta = kScoreThreads / 32;
    const size_t bar_bytes = (size_t)warps_per_cta * kMaxRingStages * 8;
    const size_t off_bytes = n_req + 1 <= kMaxSmemOffsets ? (((size_t)n_req + 1) * 4 + 15) / 16 * 16 : 0;
    // what a thread block has for its rings when `ctas` of them share an SM (1 KiB per block is the system's)
    auto ring_room = [&](int ctas) -> int64_t {
        return (int64_t)kSmemPerSm / ctas - 1024 - (int64_t)static_bytes - (int64_t)bar_bytes - (int64_t)off_bytes;
    };
    int ctas_per_sm = 2;
    int stages = (int)(ring_room(2) / (int64_t)((size_t)warps_per_cta * row_bytes));
    if (stages < 2) {                         // very wide rows: one thread block per SM gets all of it
        ctas_per_sm = 1;
        stages = (int)(ring_room(1) / (int64_t)((size_t)warps_per_cta * row_bytes));
    }
    // four buffers for rows of 2 KiB and more (more do not help: measured), eight of 1 KiB, sixteen below
    const int cap = row_bytes >= 2048 ? kRingStages : row_bytes >= 1024 ? 8 : kMaxRingStages;
    if (stages > cap) stages = cap;
    RingGeometry g;
    int64_t grid = (int64_t)sm_count() * ctas_per_sm;
    const int64_t want = ((int64_t)total + warps_per_cta - 1) / warps_per_cta;   // at least a row per warp
    if (grid > want) grid = want;
    g.grid = (int)(grid < 1 ? 1 : grid);
    g.stages = stages;
    g.smem = bar_bytes + (size_t)warps_per_cta * stages * row_bytes + off_bytes;
    return g;
}

template <int DT, int QN, bool FUSEQ, int R, bool PEER>
int32_t launch_ring_pick(ScoreParams p, cudaStream_t st);

template <int DT, int QN, bool FUSEQ, int R = 1>
int32_t launch_ring_one(const ScoreParams& p, cudaStream_t st)
{
    // (several representatives per head are scored on one rank only)
    if (R == 1 && p.px.world > 0) return launch_ring_pick<DT, QN, FUSEQ, 1, true>(p, st);
    return launch_ring_pick<DT, QN, FUSEQ, R, false>(p, st);
}

template <int DT, int QN, bool FUSEQ, int R, bool PEER>
int32_t launch_ring_pick(ScoreParams p, cudaStream_t st)
{
    constexpr uint32_t kRowBytes = (uint32_t)QN * 32u * (DT == UCMX_DT_BF16 ? 2u : 4u);
    // static shared memory of the kernel: the staged queries of the fused variant
    const size_t static_bytes = FUSEQ ? (size_t)3 * QN * 32 * 4 + 64 : 64;
    const RingGeometry g = ring_geometry(p.total, kRowBytes, p.n_req, static_bytes);
    if (g.stages < 1) return UCMX_EUNSUPPORTED;
    static int smem_set[64];                  // per device: dynamic shared memory limit already raised to this
    int dev = 0;
    UCMX_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && smem_set[dev] < (int)g.smem) {
        UCMX_CUDA(cudaFuncSetAttribute(score_dot_ring_kernel<DT, QN, FUSEQ, R, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)g.smem));
        smem_set[dev] = (int)g.smem;
    }
    p.stages = g.stages;
    const int64_t warps = (int64_t)g.grid * (kScoreThreads / 32);
    p.rows_per_warp = (int32_t)((p.total + warps - 1) / warps);
    p.d_shift = -1;
    for (int sh = 0; sh < 16; ++sh)
        if ((1 << sh) == p.D) p.d_shift = sh;
    // (ranks that exchange scores read the round counter the kernel ahead may still be writing: never early)
    p.early = early_start() && p.px.world == 0 ? 1 : 0;
    if (p.early) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)g.grid);
        cfg.blockDim = dim3(kScoreThreads);
        cfg.dynamicSmemBytes = g.smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        UCMX_CUDA(cudaLaunchKernelEx(&cfg, score_dot_ring_kernel<DT, QN, FUSEQ, R, PEER>, p));
    } else {
        score_dot_ring_kernel<DT, QN, FUSEQ, R, PEER><<<g.grid, kScoreThreads, g.smem, st>>>(p);
    }
    UCMX_LAUNCH_CHECK("score_dot_ring_kernel");
    return UCMX_OK;
}

// several representatives per head (bf16 tables of 128-channel vectors): rows of 512 B to 4 KiB
int32_t launch_ring_reps(const ScoreParams& p, int qn, int n_rep, cudaStream_t st)
{
    if (n_rep == 2) {
        switch (qn) {
            case 8: return launch_ring_one<UCMX_DT_BF16, 8, false, 2>(p, st);
            case 16: return launch_ring_one<UCMX_DT_BF16, 16, false, 2>(p, st);
            case 32: return launch_ring_one<UCMX_DT_BF16, 32, false, 2>(p, st);
            case 64: return launch_ring_one<UCMX_DT_BF16, 64, false, 2>(p, st);
            default: return UCMX_EUNSUPPORTED;
        }
    }
    if (n_rep == 4) {
        switch (qn) {
            case 16: return launch_ring_one<UCMX_DT_BF16, 16, false, 4>(p, st);
            case 32: return launch_ring_one<UCMX_DT_BF16, 32, false, 4>(p, st);
            case 64: return launch_ring_one<UCMX_DT_BF16, 64, false, 4>(p, st);
            default: return UCMX_EUNSUPPORTED;
        }
    }
    return UCMX_EUNSUPPORTED;
}

template <int DT, bool FUSEQ>
int32_t launch_ring(const ScoreParams& p, int qn, cudaStream_t st)
{
    switch (qn) {
        case 8: return launch_ring_one<DT, 8, FUSEQ>(p, st);
        case 16: return launch_ring_one<DT, 16, FUSEQ>(p, st);
        case 32: return launch_ring_one<DT, 32, FUSEQ>(p, st);
        case 64: return launch_ring_one<DT, 64, FUSEQ>(p, st);
        default: return UCMX_EUNSUPPORTED;
    }
}

bool rows_path_ok(int32_t reps_dtype, int32_t n_rep, int64_t E, int* qn)
{
    const int per_piece = reps_dtype == UCMX_DT_BF16 ? 8 : 4;
    if (n_rep != 1 || E % (32 * per_piece) != 0) return false;
    *qn = (int)(E / 32);
    return *qn == 8 || *qn == 16 || *qn == 32 || *qn == 64;
}

int rows_grid(int32_t total)
{
    // one resident wave: two CTAs of 8 warps per SM; fewer when there is less than a row per warp
    const int warps_per_cta = kScoreThreads / 32;
    int64_t grid = (int64_t)sm_count() * 2;
    const int64_t want = ((int64_t)total + warps_per_cta - 1) / warps_per_cta;
    if (grid > want) grid = want;
    return (int)(grid < 1 ? 1 : grid);
}

// Checks a ucmx_peer_exchange descriptor against the batch and turns it into the kernels' form.
int32_t peer_push_from(const ucmx_peer_exchange* ex, int32_t total, PeerPush* out)
{
    out->bases = nullptr;
    out->world = 0;
    out->my_rank = 0;
    out->part_bytes = 0;
    if (!ex) return UCMX_OK;
    if (!ex->bases || ex->world < 1 || ex->world > 32 || ex->my_rank < 0 || ex->my_rank >= ex->world ||
        ex->n_scores < total)
        return UCMX_EPARAM;
    out->bases = (unsigned char* const*)ex->bases;
    out->world = ex->world;
    out->my_rank = ex->my_rank;
    out->part_bytes = peer_part_bytes(ex->n_scores);
    return UCMX_OK;
}

// Narrow rows, one representative per head: a row of 32 to 256 bytes (for instance one KV head of 128 bf16
// channels, which is what a rank holds under eight-way head parallelism) is too short for a warp and a copy of its
// own.  Here a group of LPR lanes owns a row, a warp covers 32 / LPR rows with one load instruction and keeps up to
// sixteen such instructions (32 rows) in flight; the slot ids of an iteration's rows come in with one coalesced read, asked for
// an iteration ahead, so that a row's load never waits for its id.  Every lane walks the request boundaries for its
// own rows (they only grow) and takes its eight (bf16) or four (fp32) query elements from the L1-resident query.
template <int DT, int LPR>
__global__ void __launch_bounds__(kScoreThreads) score_dot_narrow_kernel(ScoreGenParams p)
{
    constexpr int kRows = 32 / LPR;          // rows per load instruction of a warp
    constexpr int kU = kRows * 16 <= 32 ? 16 : 32 / kRows;   // load instructions in flight (their rows' ids fit one warp-wide read)
    constexpr int kStep = kRows * kU;        // rows per iteration
    constexpr int kPer = (DT == UCMX_DT_BF16) ? 8 : 4;
    const int lane = threadIdx.x & 31, sub = lane / LPR, pc = lane % LPR;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int begin = (int)((int64_t)p.total * w / W);
    const int end = (int)((int64_t)p.total * (w + 1) / W);
    uint32_t round = 0;
    int64_t push_off = 0;
    if (p.px.world > 0) {
        round = peer_round_now(p.px);
        push_off = peer_inbox_offset(p.px, round, p.px.my_rank);
    }
    if (begin < end) {
        const int E = p.H * p.D;
        const size_t row_bytes = (size_t)E * (DT == UCMX_DT_BF16 ? 2 : 4);
        const unsigned char* base = reinterpret_cast<const unsigned char*>(p.reps);
        // slot of row c + lane for the first kStep lanes (-2: past the end, -1: an empty entry of the table)
        auto ids_of = [&](int c) -> int {
            const int row = c + lane;
            return (lane < kStep && row < end) ? checked_slot(p.slot_ids, row, p.n_slots, p.err) : -2;
        };
        int ids_next = ids_of(begin);
        int r = find_request(p.offsets, p.n_req, begin);
        int r_end = __ldg(p.offsets + r + 1);
        for (int c = begin; c < end; c += kStep) {
            const int ids = ids_next;
            ids_next = ids_of(c + kStep);
            uint4 v[kU];
            int slot[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                slot[u] = __shfl_sync(0xffffffffu, ids, u * kRows + sub);
                v[u] = make_uint4(0, 0, 0, 0);
                if (slot[u] >= 0) v[u] = ld_stream16(base + (size_t)slot[u] * row_bytes + (size_t)pc * 16);
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int row = c + u * kRows + sub;
                float acc = 0.0f;
                if (slot[u] >= 0) {
                    while (row >= r_end) {
                        ++r;
                        r_end = __ldg(p.offsets + r + 1);
                    }
                    const float4* qq = reinterpret_cast<const float4*>(p.q + (int64_t)r * E + pc * kPer);
                    const float4 q0 = __ldg(qq);
                    if (DT == UCMX_DT_BF16) {
                        const float4 q1 = __ldg(qq + 1);
                        acc = fmaf(q0.x, bf16lo(v[u].x), acc);
                        acc = fmaf(q0.y, bf16hi(v[u].x), acc);
                        acc = fmaf(q0.z, bf16lo(v[u].y), acc);
                        acc = fmaf(q0.w, bf16hi(v[u].y), acc);
                        acc = fmaf(q1.x, bf16lo(v[u].z), acc);
                        acc = fmaf(q1.y, bf16hi(v[u].z), acc);
                        acc = fmaf(q1.z, bf16lo(v[u].w), acc);
                        acc = fmaf(q1.w, bf16hi(v[u].w), acc);
                    } else {
                        acc = fmaf(q0.x, __uint_as_float(v[u].x), acc);
                        acc = fmaf(q0.y, __uint_as_float(v[u].y), acc);
                        acc = fmaf(q0.z, __uint_as_float(v[u].z), acc);
                        acc = fmaf(q0.w, __uint_as_float(v[u].w), acc);
                    }
                }
#pragma unroll
                for (int o = LPR >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (slot[u] != -2) {
                    // the lanes of a row's group all hold the score: lane pc of the group delivers to rank pc
                    // (and lane 0 to the local output), so the stores to the peers leave side by side
                    const float val = slot[u] >= 0 ? acc * p.scale : -INFINITY;
                    if (pc == 0 && p.out) p.out[row] = val;
                    for (int t = pc; t < p.px.world; t += LPR)
                        reinterpret_cast<float*>(p.px.bases[t] + push_off)[row] = val;
                }
            }
        }
    }
    if (p.px.world > 0) peer_publish_round(p.px, round);
}

template <int DT>
bool launch_narrow(const ScoreGenParams& g, int64_t row_bytes, cudaStream_t st)
{
    const int grid = rows_grid(g.total);
    switch (row_bytes) {
        case 256: score_dot_narrow_kernel<DT, 16><<<grid, kScoreThreads, 0, st>>>(g); return true;
        case 128: score_dot_narrow_kernel<DT, 8><<<grid, kScoreThreads, 0, st>>>(g); return true;
        case 64: score_dot_narrow_kernel<DT, 4><<<grid, kScoreThreads, 0, st>>>(g); return true;
        case 32: score_dot_narrow_kernel<DT, 2><<<grid, kScoreThreads, 0, st>>>(g); return true;
        default: return false;
    }
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_query_group_mean(const void* q, int32_t n_tok, int32_t n_q_heads, int32_t n_kv_heads,
                                         int32_t head_dim, int64_t tok_stride, int32_t round_bf16, float* out,
                                         ucmx_stream_t stream)
{
    using namespace ucmx;
    if (!q || !out || n_tok < 0 || n_q_heads < 1 || n_kv_heads < 1 || head_dim < 1) return UCMX_EPARAM;
    if (n_q_heads >= n_kv_heads ? (n_q_heads % n_kv_heads) : (n_kv_heads % n_q_heads)) return UCMX_EPARAM;
    if (tok_stride < (int64_t)n_q_heads * head_dim) return UCMX_EPARAM;
    if (n_tok == 0) return UCMX_OK;
    const int64_t total = (int64_t)n_tok * n_kv_heads * head_dim;
    const int threads = 256;
    const int64_t grid = (total + threads - 1) / threads;
    query_group_mean_kernel<<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>(
        (const uint16_t*)q, n_tok, n_q_heads, n_kv_heads, head_dim, tok_stride, round_bf16, out);
    UCMX_LAUNCH_CHECK("query_group_mean_kernel");
    return UCMX_OK;
}

namespace ucmx {
int32_t score_dot_impl(const void* reps, int32_t reps_dtype, int64_t n_slots, int32_t n_kv_heads, int32_t n_rep,
                       int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids, const float* q,
                       int32_t n_req, int32_t total, float scale, float* out_scores, const ucmx_peer_exchange* ex,
                       int32_t* err, cudaStream_t st)
{
    if (n_req < 0 || total < 0 || n_slots < 0) return UCMX_EPARAM;
    if (n_req == 0 || total == 0) return UCMX_OK;
    if (!reps || !req_offsets || !q || (!out_scores && !ex)) return UCMX_EPARAM;
    if (reps_dtype != UCMX_DT_BF16 && reps_dtype != UCMX_DT_F32) return UCMX_EPARAM;
    if (n_kv_heads < 1 || n_rep < 1 || head_dim < 8 || head_dim % 8) return UCMX_EPARAM;
    if (((uintptr_t)reps & 15) || ((uintptr_t)q & 15)) return UCMX_EPARAM;
    PeerPush px;
    const int32_t rc = peer_push_from(ex, total, &px);
    if (rc != UCMX_OK) return rc;
    const int64_t E = (int64_t)n_kv_heads * head_dim;
    int qn = 0;
    if (rows_path_ok(reps_dtype, n_rep, E, &qn)) {
        ScoreParams p{};
        p.reps = reps;
        p.n_slots = n_slots;
        p.offsets = req_offsets;
        p.slot_ids = slot_ids;
        p.q = q;
        p.D = head_dim;
        p.out = out_scores;
        p.n_req = n_req;
        p.total = total;
        p.E = (int32_t)E;
        p.scale = scale;
        p.px = px;
        p.err = err;
        if (reps_dtype == UCMX_DT_BF16) return launch_ring<UCMX_DT_BF16, false>(p, qn, st);
        return launch_ring<UCMX_DT_F32, false>(p, qn, st);
    }
    if (reps_dtype == UCMX_DT_BF16 && head_dim == 128 && (n_rep == 2 || n_rep == 4) && !ex) {
        // GSA's tables: the row ring with the per-head maximum over representatives folded into the reduction
        const int64_t row_elems = E * n_rep;
        const int qn_r = (int)(row_elems / 32);
        if ((qn_r == 8 || qn_r == 16 || qn_r == 32 || qn_r == 64) && (n_rep == 2 || qn_r >= 16)) {
            ScoreParams p{};
            p.reps = reps;
            p.n_slots = n_slots;
            p.offsets = req_offsets;
            p.slot_ids = slot_ids;
            p.q = q;
            p.D = head_dim;
            p.out = out_scores;
            p.n_req = n_req;
            p.total = total;
            p.E = (int32_t)E;
            p.scale = scale;
            p.px = px;
            p.err = err;
            const int32_t rr = launch_ring_reps(p, qn_r, n_rep, st);
            if (rr != UCMX_EUNSUPPORTED) return rr;
        }
    }
    ScoreGenParams g{reps, n_slots, req_offsets, slot_ids, q, out_scores, n_req, total, n_kv_heads, n_rep, head_dim, scale, px, err};
    if (n_rep == 1) {
        const int64_t row_bytes = E * (reps_dtype == UCMX_DT_BF16 ? 2 : 4);
        const bool done = reps_dtype == UCMX_DT_BF16 ? launch_narrow<UCMX_DT_BF16>(g, row_bytes, st) : launch_narrow<UCMX_DT_F32>(g, row_bytes, st);
        if (done) {
            UCMX_LAUNCH_CHECK("score_dot_narrow_kernel");
            return UCMX_OK;
        }
    }
    if (ex) {
        set_last_text("score_dot: the peer exchange is available for one representative per head and rows of 32-256 bytes "
                      "or a multiple of 512 bytes up to 4 KiB (bf16) / 8 KiB (fp32)");
        return UCMX_EUNSUPPORTED;
    }
    if (reps_dtype == UCMX_DT_BF16 && head_dim == 128) {
        // GSA's shapes: the whole row in flight (see score_dot_reps_kernel)
        int64_t g4 = (int64_t)sm_count() * 4;          // four thread blocks of 8 warps per SM: 128 KiB of rows in flight
        const int64_t want4 = ((int64_t)total + 7) / 8;
        const int grid2 = (int)(g4 < want4 ? g4 : (want4 < 1 ? 1 : want4));
        // (rows up to 4 KiB went to the row ring above: what is left is four representatives of eight heads, 8 KiB)
        bool done = true;
        if (n_rep == 4 && n_kv_heads == 8) score_dot_reps_kernel<16, 4><<<grid2, kScoreThreads, 0, st>>>(g);
        else done = false;
        if (done) {
            UCMX_LAUNCH_CHECK("score_dot_reps_kernel");
            return UCMX_OK;
        }
    }
    const int warps_per_cta = kScoreThreads / 32;
    int64_t want = ((int64_t)total + warps_per_cta - 1) / warps_per_cta;
    const int64_t cap = (int64_t)sm_count() * 8;
    int grid = (int)(want > cap ? cap : want);
    if (reps_dtype == UCMX_DT_BF16)
        score_dot_general_kernel<UCMX_DT_BF16><<<grid, kScoreThreads, 0, st>>>(g);
    else
        score_dot_general_kernel<UCMX_DT_F32><<<grid, kScoreThreads, 0, st>>>(g);
    UCMX_LAUNCH_CHECK("score_dot_general_kernel");
    return UCMX_OK;
}
}  // namespace ucmx

extern "C" int32_t ucmx_score_dot(const void* reps, int32_t reps_dtype, int64_t n_slots, int32_t n_kv_heads,
                                  int32_t n_rep, int32_t head_dim, const int32_t* req_offsets,
                                  const int32_t* slot_ids, const float* q, int32_t n_req, int32_t total, float scale,
                                  float* out_scores, const ucmx_peer_exchange* exchange, ucmx_stream_t stream)
{
    return ucmx::score_dot_impl(reps, reps_dtype, n_slots, n_kv_heads, n_rep, head_dim, req_offsets, slot_ids, q, n_req,
                                total, scale, out_scores, exchange, ucmx::error_word(), (cudaStream_t)stream);
}

namespace ucmx {
namespace {
// ---------------------------------------------------------------------------------------------
// GSA's device-side weights (cal_topk, ucm/sparse/gsa/gsa.py:386-412): per QUERY head the largest dot
// product with the block's n_rep representatives of its KV head, averaged over query heads; include
// and exclude masks turn into +inf / -inf (exclude last).  One warp per candidate.  The warp is cut into
// g = Hq/H lane groups, one per query head of the KV head at hand, so the representative row is read once
// per (head, representative) - as a broadcast - and the reduction is a short one inside the group.
struct ScoreHeadsParams {
    const void* reps;           // [slot][H][R][D] bf16
    int64_t n_slots;
    int32_t* err;
    const int32_t* offsets;
    const int32_t* slot_ids;
    const uint16_t* q;          // bf16 [n_req][Hq][D], q_stride elements between requests
    const uint8_t* include_mask;
    const uint8_t* exclude_mask;
    float* out;
    int64_t q_stride;
    int32_t n_req, total, H, Hq, R, D;
};

__global__ void __launch_bounds__(kScoreThreads) score_dot_heads_kernel(ScoreHeadsParams p)
{
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int g = p.Hq / p.H;                  // query heads per KV head: 1, 2, 4, ... 32
    const int lanes_per_head = 32 / g;
    const int gi = lane / lanes_per_head;      // which query head of the group this lane works for
    const int li = lane - gi * lanes_per_head;
    const int pieces = p.D / 4;                // 8-byte pieces of a row
    const uint16_t* reps = reinterpret_cast<const uint16_t*>(p.reps);
    const float inv = 1.0f / (float)p.Hq;

    for (int64_t c = w0; c < p.total; c += W) {
        const int r = find_request(p.offsets, p.n_req, (int)c);
        const int slot = checked_slot(p.slot_ids, c, p.n_slots, p.err);
        if (slot < 0) {
            if (lane == 0) p.out[c] = -INFINITY;
            continue;
        }
        const uint16_t* row = reps + (size_t)slot * p.H * p.R * p.D;
        const uint16_t* qr = p.q + (int64_t)r * p.q_stride;
        float total = 0.0f;                    // lane li == 0 of each group: sum over KV heads of its query head's maximum
        for (int h = 0; h < p.H; ++h) {
            const uint16_t* qv = qr + (size_t)(h * g + gi) * p.D;
            float best = -INFINITY;
            for (int j = 0; j < p.R; ++j) {
                const uint16_t* kv = row + ((size_t)h * p.R + j) * p.D;
                float acc = 0.0f;
                for (int pc = li; pc < pieces; pc += lanes_per_head) {
                    const uint2 kw = __ldg(reinterpret_cast<const uint2*>(kv) + pc);
                    const uint2 qw = __ldg(reinterpret_cast<const uint2*>(qv) + pc);
                    acc = fmaf(bf16lo(qw.x), bf16lo(kw.x), acc);
                    acc = fmaf(bf16hi(qw.x), bf16hi(kw.x), acc);
                    acc = fmaf(bf16lo(qw.y), bf16lo(kw.y), acc);
                    acc = fmaf(bf16hi(qw.y), bf16hi(kw.y), acc);
                }
                for (int o = lanes_per_head >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                best = fmaxf(best, acc);
            }
            total += best;
        }
        // one value per lane group (every lane of a group holds it): add the groups up
        for (int o = lanes_per_head; o < 32; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) {
            float w = total * inv;
            if (p.include_mask && __ldg(p.include_mask + c)) w = INFINITY;
            if (p.exclude_mask && __ldg(p.exclude_mask + c)) w = -INFINITY;
            p.out[c] = w;
        }
    }
}

// The same weights for the shapes GSA runs with - 128 channels per head, 2 or 4 representatives - with the whole row in
// flight (as in score_dot_reps_kernel): a warp-wide load brings two representative vectors, one per half-warp, and
// each half-warp takes the dot products of its vector with the G query heads of the KV head at hand (the query rows
// come from L1: a warp's candidates belong to one request for long stretches).
template <int NV, int R, int G>
__global__ void __launch_bounds__(kScoreThreads) score_dot_heads_rows_kernel(ScoreHeadsParams p)
{
    constexpr int kLoadsPerHead = R / 2;
    constexpr int kHeads = NV / kLoadsPerHead;
    const int lane = threadIdx.x & 31, pc = lane & 15;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int begin = (int)((int64_t)p.total * w / W);
    const int end = (int)((int64_t)p.total * (w + 1) / W);
    if (begin >= end) return;
    const unsigned char* base = reinterpret_cast<const unsigned char*>(p.reps);
    constexpr size_t kRowBytes = (size_t)NV * 512;
    const float inv = 1.0f / (float)(kHeads * G);
    int slot_next = checked_slot(p.slot_ids, begin, p.n_slots, p.err);
    int r = find_request(p.offsets, p.n_req, begin);
    int r_end = __ldg(p.offsets + r + 1);
    for (int c = begin; c < end; ++c) {
        const int slot = slot_next;
        if (c + 1 < end) slot_next = checked_slot(p.slot_ids, c + 1, p.n_slots, p.err);
        if (slot < 0) {
            if (lane == 0) p.out[c] = -INFINITY;
            continue;
        }
        uint4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = ld_stream16(base + (size_t)slot * kRowBytes + (size_t)i * 512 + (size_t)lane * 16);
        while (c >= r_end) {
            ++r;
            r_end = __ldg(p.offsets + r + 1);
        }
        const uint16_t* qr = p.q + (int64_t)r * p.q_stride + pc * 8;
        // Per KV head: the G x kLoadsPerHead dot products of this lane's eight channels, summed over the half-warp all
        // at once (half_warp_sums); value gi * kLoadsPerHead + j ends up in the lane whose low bits spell it, so the
        // maximum over a head's loads is taken between lanes G and more apart, the other half-warp holds the other
        // representatives, and each lane adds up the best of "its" query head over the KV heads.
        float total = 0.0f;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            float part[G * kLoadsPerHead];
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const uint4 qv = __ldg(reinterpret_cast<const uint4*>(qr + (size_t)(h * G + gi) * 128));
                const float2 qa = make_float2(bf16lo(qv.x), bf16hi(qv.x)), qb = make_float2(bf16lo(qv.y), bf16hi(qv.y));
                const float2 qc = make_float2(bf16lo(qv.z), bf16hi(qv.z)), qd = make_float2(bf16lo(qv.w), bf16hi(qv.w));
#pragma unroll
                for (int j = 0; j < kLoadsPerHead; ++j) {
                    const uint4 x = v[h * kLoadsPerHead + j];
                    float2 s0 = __fmul2_rn(qa, make_float2(bf16lo(x.x), bf16hi(x.x)));
                    float2 s1 = __fmul2_rn(qb, make_float2(bf16lo(x.y), bf16hi(x.y)));
                    s0 = __ffma2_rn(qc, make_float2(bf16lo(x.z), bf16hi(x.z)), s0);
                    s1 = __ffma2_rn(qd, make_float2(bf16lo(x.w), bf16hi(x.w)), s1);
                    part[gi * kLoadsPerHead + j] = (s0.x + s1.x) + (s0.y + s1.y);
                }
            }
            float best = half_warp_sums<G * kLoadsPerHead, 1>(part, lane);
#pragma unroll
            for (int o = G; o < G * kLoadsPerHead; o <<= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
            total += fmaxf(best, __shfl_xor_sync(0xffffffffu, best, 16));
        }
#pragma unroll
        for (int o = 1; o < G; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) {
            float wgt = total * inv;
            if (p.include_mask && __ldg(p.include_mask + c)) wgt = INFINITY;
            if (p.exclude_mask && __ldg(p.exclude_mask + c)) wgt = -INFINITY;
            p.out[c] = wgt;
        }
    }
}

template <int NV, int R>
bool launch_heads_rows(const ScoreHeadsParams& p, int g, int grid, cudaStream_t st)
{
    switch (g) {
        case 1: score_dot_heads_rows_kernel<NV, R, 1><<<grid, kScoreThreads, 0, st>>>(p); return true;
        case 2: score_dot_heads_rows_kernel<NV, R, 2><<<grid, kScoreThreads, 0, st>>>(p); return true;
        case 4: score_dot_heads_rows_kernel<NV, R, 4><<<grid, kScoreThreads, 0, st>>>(p); return true;
        case 8: score_dot_heads_rows_kernel<NV, R, 8><<<grid, kScoreThreads, 0, st>>>(p); return true;
        default: return false;
    }
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_score_dot_heads(const void* reps, int64_t n_slots, int32_t n_kv_heads, int32_t n_rep,
                                        int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids, const void* query,
                                        int32_t n_q_heads, int64_t query_stride, int32_t n_req, int32_t total,
                                        const uint8_t* include_mask, const uint8_t* exclude_mask, float* out_scores,
                                        ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_req < 0 || total < 0 || n_slots < 0) return UCMX_EPARAM;
    if (n_req == 0 || total == 0) return UCMX_OK;
    if (!reps || !req_offsets || !query || !out_scores) return UCMX_EPARAM;
    if (n_kv_heads < 1 || n_rep < 1 || head_dim < 4 || (head_dim & 3) || n_q_heads < n_kv_heads || n_q_heads % n_kv_heads) return UCMX_EPARAM;
    const int g = n_q_heads / n_kv_heads;
    if (g > 32 || (g & (g - 1))) {
        set_last_text("score_dot_heads: query heads per KV head must be a power of two up to 32");
        return UCMX_EUNSUPPORTED;
    }
    if (query_stride < (int64_t)n_q_heads * head_dim || (query_stride & 3) || ((uintptr_t)reps & 7) || ((uintptr_t)query & 7)) return UCMX_EPARAM;
    ScoreHeadsParams p{};
    p.reps = reps;
    p.n_slots = n_slots;
    p.err = error_word();
    p.offsets = req_offsets;
    p.slot_ids = slot_ids;
    p.q = (const uint16_t*)query;
    p.include_mask = include_mask;
    p.exclude_mask = exclude_mask;
    p.out = out_scores;
    p.q_stride = query_stride;
    p.n_req = n_req;
    p.total = total;
    p.H = n_kv_heads;
    p.Hq = n_q_heads;
    p.R = n_rep;
    p.D = head_dim;
    const int warps_per_cta = kScoreThreads / 32;
    int64_t want = ((int64_t)total + warps_per_cta - 1) / warps_per_cta;
    if (head_dim == 128 && (query_stride % 8) == 0 && !((uintptr_t)reps & 15) && !((uintptr_t)query & 15)) {
        // GSA's shapes: the whole row in flight
        const int64_t cap4 = (int64_t)sm_count() * 3;
        const int grid = (int)(want > cap4 ? cap4 : want);
        bool done = false;
        if (n_rep == 2 && n_kv_heads == 8) done = launch_heads_rows<8, 2>(p, g, grid, (cudaStream_t)stream);
        else if (n_rep == 2 && n_kv_heads == 4) done = launch_heads_rows<4, 2>(p, g, grid, (cudaStream_t)stream);
        else if (n_rep == 2 && n_kv_heads == 2) done = launch_heads_rows<2, 2>(p, g, grid, (cudaStream_t)stream);
        else if (n_rep == 2 && n_kv_heads == 1) done = launch_heads_rows<1, 2>(p, g, grid, (cudaStream_t)stream);
        else if (n_rep == 4 && n_kv_heads == 8) done = launch_heads_rows<16, 4>(p, g, grid, (cudaStream_t)stream);
        else if (n_rep == 4 && n_kv_heads == 4) done = launch_heads_rows<8, 4>(p, g, grid, (cudaStream_t)stream);
        if (done) {
            UCMX_LAUNCH_CHECK("score_dot_heads_rows_kernel");
            return UCMX_OK;
        }
    }
    const int64_t cap = (int64_t)sm_count() * 8;
    score_dot_heads_kernel<<<(int)(want > cap ? cap : want), kScoreThreads, 0, (cudaStream_t)stream>>>(p);
    UCMX_LAUNCH_CHECK("score_dot_heads_kernel");
    return UCMX_OK;
}

extern "C" int32_t ucmx_score_dot_query(const void* reps, int32_t reps_dtype, int64_t n_slots, int32_t n_kv_heads,
                                        int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids,
                                        const void* query, int32_t n_q_heads, int64_t query_stride, int32_t round_bf16,
                                        int32_t n_req, int32_t total, float scale, float* out_scores,
                                        const ucmx_peer_exchange* exchange, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_req < 0 || total < 0 || n_slots < 0) return UCMX_EPARAM;
    if (n_req == 0 || total == 0) return UCMX_OK;
    if (!reps || !req_offsets || !query || (!out_scores && !exchange)) return UCMX_EPARAM;
    if (reps_dtype != UCMX_DT_BF16 && reps_dtype != UCMX_DT_F32) return UCMX_EPARAM;
    if (n_kv_heads < 1 || n_q_heads < 1 || head_dim < 8 || head_dim % 8) return UCMX_EPARAM;
    if (n_q_heads >= n_kv_heads ? (n_q_heads % n_kv_heads) : (n_kv_heads % n_q_heads)) return UCMX_EPARAM;
    if (query_stride < (int64_t)n_q_heads * head_dim || (query_stride % 4)) return UCMX_EPARAM;
    if (((uintptr_t)reps & 15) || ((uintptr_t)query & 7)) return UCMX_EPARAM;
    const int64_t E = (int64_t)n_kv_heads * head_dim;
    int qn = 0;
    if (!rows_path_ok(reps_dtype, 1, E, &qn)) return UCMX_EUNSUPPORTED;
    ScoreParams p{};
    const int32_t rc = peer_push_from(exchange, total, &p.px);
    if (rc != UCMX_OK) return rc;
    p.reps = reps;
    p.n_slots = n_slots;
    p.offsets = req_offsets;
    p.slot_ids = slot_ids;
    p.q_raw = (const uint16_t*)query;
    p.q_raw_stride = query_stride;
    p.Hq = n_q_heads;
    p.D = head_dim;
    p.round_bf16 = round_bf16;
    p.out = out_scores;
    p.n_req = n_req;
    p.total = total;
    p.E = (int32_t)E;
    p.scale = scale;
    p.err = error_word();
    if (reps_dtype == UCMX_DT_BF16) return launch_ring<UCMX_DT_BF16, true>(p, qn, (cudaStream_t)stream);
    return launch_ring<UCMX_DT_F32, true>(p, qn, (cudaStream_t)stream);
}

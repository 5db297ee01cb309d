// Stage 2: query-to-block scoring over a ragged batch of decode requests.
//
// score_dot: every candidate block contributes one table row (2 KiB of bf16 for 8 heads x 128)
// that is read exactly once and dotted with its request's query, so the kernel is a gather-GEMV
// bound by HBM (about 1 flop per byte); it runs on CUDA cores with 16-byte streaming loads, one
// warp per row, the query held in registers.  Tensor cores would add nothing here.
#include "common.cuh"

namespace ucmx {
namespace {

constexpr int kScoreThreads = 256;
constexpr int kMaxSmemOffsets = 2049;

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
    const int32_t* offsets;
    const int32_t* slot_ids;
    const float* q;
    float* out;
    int32_t n_req, total, E;
    float scale;
};

// Element layout per lane: a row is cut into 16-byte pieces; piece j of a row belongs to lane
// j % 32.  A piece holds 8 bf16 or 4 fp32 values.  QN = E/32 values of q per lane.
template <int DT, int QN>
struct RowDot {
    static constexpr int kPerPiece = (DT == UCMX_DT_BF16) ? 8 : 4;
    static constexpr int kPieces = QN / kPerPiece;

    float q[QN];

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
    __device__ __forceinline__ float dot(const uint4 (&buf)[kPieces]) const
    {
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

template <int DT, int QN>
__global__ void __launch_bounds__(kScoreThreads) score_dot_rows_kernel(ScoreParams p)
{
    __shared__ int32_t s_off[kMaxSmemOffsets];
    const bool off_in_smem = p.n_req + 1 <= kMaxSmemOffsets;
    if (off_in_smem) {
        for (int i = threadIdx.x; i <= p.n_req; i += blockDim.x) s_off[i] = __ldg(p.offsets + i);
        __syncthreads();
    }
    const int32_t* off = off_in_smem ? s_off : p.offsets;

    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int begin = (int)((int64_t)p.total * w / W);
    const int end = (int)((int64_t)p.total * (w + 1) / W);
    if (begin >= end) return;

    using RD = RowDot<DT, QN>;
    RD rd;
    const size_t row_bytes = (size_t)p.E * (DT == UCMX_DT_BF16 ? 2 : 4);
    const unsigned char* base = reinterpret_cast<const unsigned char*>(p.reps);

    int r = 0;
    {
        int lo = 0, hi = p.n_req;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (off[mid] <= begin) lo = mid; else hi = mid;
        }
        r = lo;
    }
    int r_end = off[r + 1];
    rd.load_q(p.q + (int64_t)r * p.E, lane);

    for (int c0 = begin; c0 < end; c0 += 32) {
        // the slots of up to 32 candidates, one per lane
        const int nc = min(32, end - c0);
        int my_slot = 0;
        if (lane < nc) my_slot = p.slot_ids ? __ldg(p.slot_ids + c0 + lane) : (c0 + lane);
        int j = 0;
        for (; j + 1 < nc; j += 2) {
            const int sa = __shfl_sync(0xffffffffu, my_slot, j);
            const int sb = __shfl_sync(0xffffffffu, my_slot, j + 1);
            uint4 a[RD::kPieces], b[RD::kPieces];
            if (sa >= 0) rd.load_row(base + (size_t)sa * row_bytes, lane, a);
            else rd.zero_row(a);
            if (sb >= 0) rd.load_row(base + (size_t)sb * row_bytes, lane, b);
            else rd.zero_row(b);
            const int ca = c0 + j, cb = ca + 1;
            while (ca >= r_end) {
                ++r;
                r_end = off[r + 1];
                if (ca < r_end) rd.load_q(p.q + (int64_t)r * p.E, lane);
            }
            float va = rd.dot(a);
            if (cb >= r_end) {
                while (cb >= r_end) {
                    ++r;
                    r_end = off[r + 1];
                }
                rd.load_q(p.q + (int64_t)r * p.E, lane);
            }
            float vb = rd.dot(b);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                va += __shfl_xor_sync(0xffffffffu, va, o);
                vb += __shfl_xor_sync(0xffffffffu, vb, o);
            }
            if (lane == 0) {
                p.out[ca] = sa < 0 ? -INFINITY : va * p.scale;
                p.out[cb] = sb < 0 ? -INFINITY : vb * p.scale;
            }
        }
        if (j < nc) {
            const int sa = __shfl_sync(0xffffffffu, my_slot, j);
            uint4 a[RD::kPieces];
            if (sa >= 0) rd.load_row(base + (size_t)sa * row_bytes, lane, a);
            else rd.zero_row(a);
            const int ca = c0 + j;
            if (ca >= r_end) {
                while (ca >= r_end) {
                    ++r;
                    r_end = off[r + 1];
                }
                rd.load_q(p.q + (int64_t)r * p.E, lane);
            }
            float va = warp_sum(rd.dot(a));
            if (lane == 0) p.out[ca] = sa < 0 ? -INFINITY : va * p.scale;
        }
    }
}

// ------------------------------------------------------------------ general path: any n_rep

struct ScoreGenParams {
    const void* reps;
    const int32_t* offsets;
    const int32_t* slot_ids;
    const float* q;
    float* out;
    int32_t n_req, total, H, R, D;
    float scale;
};

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
        const int slot = p.slot_ids ? __ldg(p.slot_ids + c) : (int)c;
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

template <int DT>
int32_t launch_rows(const ScoreParams& p, int qn, int grid, cudaStream_t st)
{
    switch (qn) {
#define UCMX_ROWS_CASE(Q) \
    case Q: score_dot_rows_kernel<DT, Q><<<grid, kScoreThreads, 0, st>>>(p); break;
        UCMX_ROWS_CASE(8)
        UCMX_ROWS_CASE(16)
        UCMX_ROWS_CASE(32)
        UCMX_ROWS_CASE(64)
#undef UCMX_ROWS_CASE
        default: return UCMX_EUNSUPPORTED;
    }
    UCMX_LAUNCH_CHECK("score_dot_rows_kernel");
    return UCMX_OK;
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

extern "C" int32_t ucmx_score_dot(const void* reps, int32_t reps_dtype, int32_t n_kv_heads, int32_t n_rep,
                                  int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids,
                                  const float* q, int32_t n_req, int32_t total, float scale, float* out_scores,
                                  ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_req < 0 || total < 0) return UCMX_EPARAM;
    if (n_req == 0 || total == 0) return UCMX_OK;
    if (!reps || !req_offsets || !q || !out_scores) return UCMX_EPARAM;
    if (reps_dtype != UCMX_DT_BF16 && reps_dtype != UCMX_DT_F32) return UCMX_EPARAM;
    if (n_kv_heads < 1 || n_rep < 1 || head_dim < 8 || head_dim % 8) return UCMX_EPARAM;
    if (((uintptr_t)reps & 15) || ((uintptr_t)q & 15)) return UCMX_EPARAM;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t E = (int64_t)n_kv_heads * head_dim;
    const int per_piece = reps_dtype == UCMX_DT_BF16 ? 8 : 4;
    const int sms = sm_count();

    if (n_rep == 1 && E % (32 * per_piece) == 0) {
        const int qn = (int)(E / 32);
        if (qn == 8 || qn == 16 || qn == 32 || qn == 64) {
            ScoreParams p{reps, req_offsets, slot_ids, q, out_scores, n_req, total, (int32_t)E, scale};
            // aim at >= 2 candidates per warp, at most 8 resident CTAs per SM
            const int warps_per_cta = kScoreThreads / 32;
            int64_t want = ((int64_t)total + 2 * warps_per_cta - 1) / (2 * warps_per_cta);
            int grid = (int)(want < 1 ? 1 : (want > (int64_t)sms * 8 ? (int64_t)sms * 8 : want));
            if (reps_dtype == UCMX_DT_BF16) return launch_rows<UCMX_DT_BF16>(p, qn, grid, st);
            return launch_rows<UCMX_DT_F32>(p, qn, grid, st);
        }
    }
    ScoreGenParams g{reps, req_offsets, slot_ids, q, out_scores, n_req, total, n_kv_heads, n_rep, head_dim, scale};
    const int warps_per_cta = kScoreThreads / 32;
    int64_t want = ((int64_t)total + warps_per_cta - 1) / warps_per_cta;
    int grid = (int)(want > (int64_t)sms * 8 ? (int64_t)sms * 8 : want);
    if (reps_dtype == UCMX_DT_BF16)
        score_dot_general_kernel<UCMX_DT_BF16><<<grid, kScoreThreads, 0, st>>>(g);
    else
        score_dot_general_kernel<UCMX_DT_F32><<<grid, kScoreThreads, 0, st>>>(g);
    UCMX_LAUNCH_CHECK("score_dot_general_kernel");
    return UCMX_OK;
}

// Stage 1a: per-block key representatives by pooling over the tokens of a paged KV block.
//
// HBM-bound streaming reduction: a block of 128 tokens x 1024 bf16 is 256 KiB read for 2 KiB
// written.  Each CTA walks whole blocks; one elected thread keeps a ring of bulk async copies
// (cp.async.bulk, completion on an mbarrier) in flight from the paged cache into shared memory,
// and every thread owns 8 adjacent columns that it accumulates in fp32 in token order, which is
// the summation order of the reference's VectorMeanImpl
// (ucm/sparse/gsa/offload_ops/src/vec_product.cpp:349-387), so the fp32 mean is reproducible bit
// for bit.  The bf16 rounding the reference applies (ucm/sparse/esa/esa.py:265-266) is fused into
// the store.
#include "common.cuh"

namespace ucmx {

namespace {

constexpr int kStages = 4;
constexpr int kStageBytes = 16384;
constexpr int kMaxColGroupsPerThread = 4;

struct PoolParams {
    const uint16_t* k;
    int64_t block_stride;  // elements
    int64_t token_stride;  // elements
    int32_t T, H, D, E;    // tokens per block, heads, head dim, E = H*D
    const int32_t* ids;
    const int32_t* out_slots;
    int32_t n;
    int32_t round_bf16;
    int32_t n_rep, rep_index;
    uint16_t* out_bf16;
    float* out_f32;
    int32_t rows_per_stage;
    int32_t chunks_per_block;
    int32_t dense;  // token_stride == E: one bulk copy per stage
    int32_t* err;
};

template <int MODE>
__device__ __forceinline__ float pool_init()
{
    if (MODE == UCMX_POOL_MAX) return -INFINITY;
    if (MODE == UCMX_POOL_MIN) return INFINITY;
    return 0.0f;
}
template <int MODE>
__device__ __forceinline__ float pool_op(float a, float v)
{
    if (MODE == UCMX_POOL_MAX) return v > a ? v : a;
    if (MODE == UCMX_POOL_MIN) return v < a ? v : a;
    return a + v;
}

template <int MODE, int CGT>
__global__ void __launch_bounds__(CGT == 4 ? 1024 : 256) pool_blocks_kernel(PoolParams p)
{
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);  // kStages barriers
    unsigned char* ring = smem + 128;
    __shared__ int s_failed;

    const int tid = threadIdx.x;
    const int n_cg = p.E / 8;  // 16-byte column groups per token row
    const uint32_t row_bytes = (uint32_t)p.E * 2u;

    // blocks this CTA owns: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int my_blocks = (p.n - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total_chunks = my_blocks * p.chunks_per_block;

    if (tid == 0) {
        s_failed = 0;
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
    }
    __syncthreads();

    auto issue = [&](int g) {
        // chunk g of this CTA -> stage g % kStages
        const int lb = g / p.chunks_per_block;
        const int c = g - lb * p.chunks_per_block;
        const int blk = (int)blockIdx.x + lb * (int)gridDim.x;
        const int id = __ldg(p.ids + blk);
        const int t0 = c * p.rows_per_stage;
        const int rows = min(p.rows_per_stage, p.T - t0);
        const int s = g % kStages;
        unsigned char* dst = ring + (size_t)s * kStageBytes;
        const uint16_t* src = p.k + (int64_t)id * p.block_stride + (int64_t)t0 * p.token_stride;
        mbar_expect_tx(&full[s], (uint32_t)rows * row_bytes);
        if (p.dense) {
            bulk_g2s(dst, src, (uint32_t)rows * row_bytes, &full[s]);
        } else {
            for (int r = 0; r < rows; ++r)
                bulk_g2s(dst + (size_t)r * row_bytes, src + (int64_t)r * p.token_stride, row_bytes, &full[s]);
        }
    };

    if (tid == 0) {
        const int pre = min(kStages, total_chunks);
        for (int g = 0; g < pre; ++g) issue(g);
    }

    float acc[CGT][8];
#pragma unroll
    for (int j = 0; j < CGT; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = pool_init<MODE>();

    const float inv = 1.0f / (float)p.T;

    for (int g = 0; g < total_chunks; ++g) {
        const int s = g % kStages;
        const uint32_t parity = (uint32_t)(g / kStages) & 1u;
        const int lb = g / p.chunks_per_block;
        const int c = g - lb * p.chunks_per_block;
        const int rows = min(p.rows_per_stage, p.T - c * p.rows_per_stage);

        bool ok = true;
        if (!s_failed) ok = mbar_wait(&full[s], parity);
        if (!ok) {
            s_failed = 1;
            if (p.err) atomicExch(p.err, 1);
        }
        const unsigned char* src = ring + (size_t)s * kStageBytes;
#pragma unroll
        for (int j = 0; j < CGT; ++j) {
            const int cg = tid + j * (int)blockDim.x;
            if (cg < n_cg) {
                const unsigned char* col = src + (size_t)cg * 16;
#pragma unroll 4
                for (int r = 0; r < rows; ++r) {
                    const uint4 v = *reinterpret_cast<const uint4*>(col + (size_t)r * row_bytes);
                    acc[j][0] = pool_op<MODE>(acc[j][0], bf16lo(v.x));
                    acc[j][1] = pool_op<MODE>(acc[j][1], bf16hi(v.x));
                    acc[j][2] = pool_op<MODE>(acc[j][2], bf16lo(v.y));
                    acc[j][3] = pool_op<MODE>(acc[j][3], bf16hi(v.y));
                    acc[j][4] = pool_op<MODE>(acc[j][4], bf16lo(v.z));
                    acc[j][5] = pool_op<MODE>(acc[j][5], bf16hi(v.z));
                    acc[j][6] = pool_op<MODE>(acc[j][6], bf16lo(v.w));
                    acc[j][7] = pool_op<MODE>(acc[j][7], bf16hi(v.w));
                }
            }
        }
        __syncthreads();  // every thread is done with stage s
        if (tid == 0 && !s_failed && g + kStages < total_chunks) issue(g + kStages);

        if (c == p.chunks_per_block - 1) {
            // block finished: finalise and store
            const int blk = (int)blockIdx.x + lb * (int)gridDim.x;
            const int64_t slot = p.out_slots ? (int64_t)__ldg(p.out_slots + blk) : (int64_t)blk;
#pragma unroll
            for (int j = 0; j < CGT; ++j) {
                const int cg = tid + j * (int)blockDim.x;
                if (cg < n_cg && slot >= 0) {
                    const int e0 = cg * 8;
                    const int h = e0 / p.D, d = e0 - h * p.D;
                    const int64_t o = ((slot * p.H + h) * p.n_rep + p.rep_index) * (int64_t)p.D + d;
                    float r[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float v = acc[j][e];
                        if (MODE == UCMX_POOL_MEAN) v *= inv;
                        r[e] = v;
                    }
                    uint32_t b[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) b[e] = f32_to_bf16_bits(r[e]);
                    if (p.out_bf16) {
                        uint4 w;
                        w.x = b[0] | (b[1] << 16);
                        w.y = b[2] | (b[3] << 16);
                        w.z = b[4] | (b[5] << 16);
                        w.w = b[6] | (b[7] << 16);
                        *reinterpret_cast<uint4*>(p.out_bf16 + o) = w;
                    }
                    if (p.out_f32) {
                        float4 f0, f1;
                        if (p.round_bf16) {
                            f0 = make_float4(__uint_as_float(b[0] << 16), __uint_as_float(b[1] << 16),
                                             __uint_as_float(b[2] << 16), __uint_as_float(b[3] << 16));
                            f1 = make_float4(__uint_as_float(b[4] << 16), __uint_as_float(b[5] << 16),
                                             __uint_as_float(b[6] << 16), __uint_as_float(b[7] << 16));
                        } else {
                            f0 = make_float4(r[0], r[1], r[2], r[3]);
                            f1 = make_float4(r[4], r[5], r[6], r[7]);
                        }
                        *reinterpret_cast<float4*>(p.out_f32 + o) = f0;
                        *reinterpret_cast<float4*>(p.out_f32 + o + 4) = f1;
                    }
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[j][e] = pool_init<MODE>();
            }
        }
    }

    // After a failed wait copies may still be in flight into this CTA's shared memory: give each
    // pending stage one more bounded wait before the memory is released.
    if (s_failed && tid == 0) {
        for (int s = 0; s < kStages; ++s) (void)mbar_wait(&full[s], 0), (void)mbar_wait(&full[s], 1);
    }
}

template <int MODE>
int32_t launch_pool(const PoolParams& p, int threads, int cgt, int grid, size_t smem, cudaStream_t st)
{
#define UCMX_POOL_CASE(C)                                                                           \
    case C: {                                                                                       \
        auto kern = pool_blocks_kernel<MODE, C>;                                                    \
        UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<grid, threads, smem, st>>>(p);                                                       \
    } break;
    switch (cgt) {
        UCMX_POOL_CASE(1)
        UCMX_POOL_CASE(2)
        UCMX_POOL_CASE(4)
        default: return UCMX_EUNSUPPORTED;
    }
#undef UCMX_POOL_CASE
    UCMX_LAUNCH_CHECK("pool_blocks_kernel");
    return UCMX_OK;
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_pool_blocks(const void* k_cache, const ucmx_kv_geometry* g, const int32_t* block_ids,
                                    const int32_t* out_slots, int32_t n, int32_t mode, int32_t round_bf16,
                                    int32_t n_rep, int32_t rep_index, void* out_bf16, float* out_f32,
                                    ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n < 0) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (!k_cache || !g || !block_ids || (!out_bf16 && !out_f32)) return UCMX_EPARAM;
    if (mode < 0 || mode > 3 || n_rep < 1 || rep_index < 0 || rep_index >= n_rep) return UCMX_EPARAM;
    if (g->block_tokens < 1 || g->n_kv_heads < 1 || g->head_dim < 8 || g->head_dim % 8) return UCMX_EPARAM;
    const int64_t E64 = (int64_t)g->n_kv_heads * g->head_dim;
    if (g->token_stride < E64 || g->token_stride % 8 || g->block_stride % 8) return UCMX_EPARAM;
    if (((uintptr_t)k_cache & 15) || ((uintptr_t)out_bf16 & 15) || ((uintptr_t)out_f32 & 15)) return UCMX_EPARAM;
    if (E64 * 2 > kStageBytes) return UCMX_EUNSUPPORTED;  // one token row must fit a stage
    if (out_bf16 && !round_bf16 && !out_f32) {
        // a bf16 table is by definition rounded
        round_bf16 = 1;
    }

    PoolParams p;
    p.k = (const uint16_t*)k_cache;
    p.block_stride = g->block_stride;
    p.token_stride = g->token_stride;
    p.T = g->block_tokens;
    p.H = g->n_kv_heads;
    p.D = g->head_dim;
    p.E = (int32_t)E64;
    p.ids = block_ids;
    p.out_slots = out_slots;
    p.n = n;
    p.round_bf16 = round_bf16;
    p.n_rep = n_rep;
    p.rep_index = rep_index;
    p.out_bf16 = (uint16_t*)out_bf16;
    p.out_f32 = out_f32;
    p.rows_per_stage = (int32_t)(kStageBytes / (E64 * 2));
    if (p.rows_per_stage > p.T) p.rows_per_stage = p.T;
    p.chunks_per_block = (p.T + p.rows_per_stage - 1) / p.rows_per_stage;
    p.dense = (g->token_stride == E64) ? 1 : 0;
    p.err = error_word();

    const int n_cg = p.E / 8;
    int threads = ((n_cg + 31) / 32) * 32;
    int cgt = 1;
    while (threads > 256 && cgt < kMaxColGroupsPerThread) {
        cgt *= 2;
        threads = (((n_cg + cgt - 1) / cgt + 31) / 32) * 32;
    }
    if (threads > 1024) return UCMX_EUNSUPPORTED;
    const size_t smem = 128 + (size_t)kStages * kStageBytes;
    const int ctas_per_sm = 3;
    int grid = sm_count() * ctas_per_sm;
    if (grid > n) grid = n;

    cudaStream_t st = (cudaStream_t)stream;
    switch (mode) {
        case UCMX_POOL_MEAN: return launch_pool<UCMX_POOL_MEAN>(p, threads, cgt, grid, smem, st);
        case UCMX_POOL_MAX: return launch_pool<UCMX_POOL_MAX>(p, threads, cgt, grid, smem, st);
        case UCMX_POOL_MIN: return launch_pool<UCMX_POOL_MIN>(p, threads, cgt, grid, smem, st);
        default: return launch_pool<UCMX_POOL_SUM>(p, threads, cgt, grid, smem, st);
    }
}

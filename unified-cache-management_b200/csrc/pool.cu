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
#include <cuda.h>

#include <cstdlib>
#include <mutex>

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
    int64_t cache_blocks;  // blocks in the cache: ids at or beyond it are dropped and reported
    int64_t out_rows;      // rows of the output table
    int32_t n;
    int32_t round_bf16;
    int32_t n_rep, rep_index;
    uint16_t* out_bf16;
    float* out_f32;
    int32_t rows_per_stage;
    int32_t chunks_per_block;
    int32_t dense;  // token_stride == E and no column split: one bulk copy per stage
    int32_t stages;      // ring depth actually used (<= kStages)
    int32_t cs;          // column splits: a block's row is cut into cs pieces, one work item each
    int32_t cg_per_item; // 16-byte column groups per work item
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
    if (MODE == UCMX_POOL_MAX) return fmaxf(a, v);  // one FMNMX; inputs are finite bf16 values
    if (MODE == UCMX_POOL_MIN) return fminf(a, v);
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
    const int n_cg = p.cg_per_item;  // 16-byte column groups of a token row this CTA reduces
    const uint32_t row_bytes = (uint32_t)n_cg * 16u;

    // work items (block, column split) this CTA owns: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int n_items = p.n * p.cs;
    const int my_items = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total_chunks = my_items * p.chunks_per_block;

    if (tid == 0) {
        s_failed = 0;
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
    }
    __syncthreads();
    const int n_stages = p.stages;

    // Called by every lane of warp 0.  Chunk g of this CTA goes to stage g % kStages.
    auto issue = [&](int g) {
        const int li = g / p.chunks_per_block;
        const int c = g - li * p.chunks_per_block;
        const int item = (int)blockIdx.x + li * (int)gridDim.x;
        const int blk = item / p.cs, split = item - blk * p.cs;
        int id = checked_block_id(p.ids, blk, p.cache_blocks, p.err);
        if (id < 0) id = 0;              // a dropped entry streams block 0 (its result is not stored)
        const int t0 = c * p.rows_per_stage;
        const int rows = min(p.rows_per_stage, p.T - t0);
        const int s = g % n_stages;
        unsigned char* dst = ring + (size_t)s * kStageBytes;
        const uint16_t* src = p.k + (int64_t)id * p.block_stride + (int64_t)t0 * p.token_stride +
                              (int64_t)split * p.cg_per_item * 8;
        if (tid == 0) mbar_expect_tx(&full[s], (uint32_t)rows * row_bytes);
        __syncwarp();
        if (p.dense) {
            if (tid == 0) bulk_g2s(dst, src, (uint32_t)rows * row_bytes, &full[s]);
        } else {
            for (int r = tid; r < rows; r += 32)
                bulk_g2s(dst + (size_t)r * row_bytes, src + (int64_t)r * p.token_stride, row_bytes, &full[s]);
        }
    };

    if (tid < 32) {
        const int pre = min(n_stages, total_chunks);
        for (int g = 0; g < pre; ++g) issue(g);
    }

    float acc[CGT][8];
#pragma unroll
    for (int j = 0; j < CGT; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = pool_init<MODE>();

    const float inv = 1.0f / (float)p.T;

    for (int g = 0; g < total_chunks; ++g) {
        const int s = g % n_stages;
        const uint32_t parity = (uint32_t)(g / n_stages) & 1u;
        const int li = g / p.chunks_per_block;
        const int c = g - li * p.chunks_per_block;
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
        if (tid < 32 && !s_failed && g + n_stages < total_chunks) issue(g + n_stages);

        if (c == p.chunks_per_block - 1) {
            // block finished: finalise and store
            const int item = (int)blockIdx.x + li * (int)gridDim.x;
            const int blk = item / p.cs, split = item - blk * p.cs;
            const int64_t slot = checked_block_id(p.ids, blk, p.cache_blocks, nullptr) < 0
                                     ? -1 : checked_out_row(p.out_slots, blk, p.out_rows, p.err);
#pragma unroll
            for (int j = 0; j < CGT; ++j) {
                const int cg = tid + j * (int)blockDim.x;
                if (cg < n_cg && slot >= 0) {
                    const int e0 = (split * p.cg_per_item + cg) * 8;
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

// ------------------------------------------------------------------ small batches: one TMA tile per CTA
//
// A decode step pools one freshly filled block per request: a few dozen blocks, far too few to
// fill the machine one block per CTA, and latency, not bandwidth, is what counts.  Here a block is
// cut into column pieces of at most 256 elements; each CTA brings its [block_tokens x piece] tile
// into shared memory with a single tiled TMA load (cp.async.bulk.tensor.3d over a tensor map of the
// paged cache: columns, tokens, blocks) and every thread owns two adjacent columns, which it sums
// in token order exactly as the streaming kernel does.

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    });
    return fn;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, int x, int y, int z, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(smem_u32(smem_dst)),
        "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(128) pool_blocks_tile_kernel(const __grid_constant__ CUtensorMap tmap, PoolParams p)
{
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
    unsigned char* tile = smem + 128;
    const int tid = threadIdx.x;
    const int cols = p.cg_per_item * 8;  // elements per piece
    const int item = blockIdx.x;
    const int blk = item / p.cs, split = item - blk * p.cs;
    const int id_in = checked_block_id(p.ids, blk, p.cache_blocks, p.err);
    const int id = id_in < 0 ? 0 : id_in;
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
        mbar_expect_tx(bar, (uint32_t)cols * 2u * (uint32_t)p.T);
        // x is a multiple of 8 elements: the 16-byte start alignment tiled TMA needs
        tma_load_3d(tile, &tmap, split * cols, 0, id, bar);
    }
    __syncthreads();
    bool ok = mbar_wait(bar, 0);
    if (!ok && p.err) atomicExch(p.err, 1);
    const int c2 = tid * 2;  // this thread's column pair inside the piece
    if (ok && c2 < cols) {
        float a0 = pool_init<MODE>(), a1 = pool_init<MODE>();
        const unsigned char* col = tile + (size_t)c2 * 2;
        const size_t pitch = (size_t)cols * 2;
#pragma unroll 8
        for (int t = 0; t < p.T; ++t) {
            const uint32_t v = *reinterpret_cast<const uint32_t*>(col + (size_t)t * pitch);
            a0 = pool_op<MODE>(a0, bf16lo(v));
            a1 = pool_op<MODE>(a1, bf16hi(v));
        }
        if (MODE == UCMX_POOL_MEAN) {
            const float inv = 1.0f / (float)p.T;
            a0 *= inv;
            a1 *= inv;
        }
        const int64_t slot = id_in < 0 ? -1 : checked_out_row(p.out_slots, blk, p.out_rows, p.err);
        if (slot >= 0) {
            const int e0 = split * cols + c2;
            const int h = e0 / p.D, d = e0 - h * p.D;
            const int64_t o = ((slot * p.H + h) * p.n_rep + p.rep_index) * (int64_t)p.D + d;
            const uint32_t b0 = f32_to_bf16_bits(a0), b1 = f32_to_bf16_bits(a1);
            if (p.out_bf16) *reinterpret_cast<uint32_t*>(p.out_bf16 + o) = b0 | (b1 << 16);
            if (p.out_f32) {
                float2 f = p.round_bf16 ? make_float2(__uint_as_float(b0 << 16), __uint_as_float(b1 << 16))
                                        : make_float2(a0, a1);
                *reinterpret_cast<float2*>(p.out_f32 + o) = f;
            }
        }
    }
    if (!ok && tid == 0) (void)mbar_wait(bar, 0);  // one more bounded wait before the tile memory is released
}

// Returns UCMX_EUNSUPPORTED when the tile path does not apply (the caller then streams).
int32_t launch_pool_tile(PoolParams& p, const ucmx_kv_geometry* g, int mode, cudaStream_t st)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc || g->reserved <= 0 || p.T > 256 || (p.D & 1)) return UCMX_EUNSUPPORTED;
    const int sms = sm_count();
    // piece width: at most 256 elements (the TMA box limit), as narrow as 64 while the grid is small
    int cs = 1;
    while (p.E / cs > 256 || ((int64_t)p.n * cs < 4 * (int64_t)sms && p.E / (cs * 2) >= 64)) {
        if (p.E % (cs * 2) || (p.E / (cs * 2)) % 8) break;
        cs *= 2;
    }
    const int cols = p.E / cs;
    if (cols > 256 || cols % 8 || p.E % cs) return UCMX_EUNSUPPORTED;
    if ((int64_t)p.n * cs > 8 * (int64_t)sms) return UCMX_EUNSUPPORTED;  // large batches stream instead
    const size_t tile_bytes = (size_t)cols * 2 * p.T;
    const size_t smem = 128 + tile_bytes;
    if (smem > 200 * 1024) return UCMX_EUNSUPPORTED;

    alignas(64) CUtensorMap tmap;
    const cuuint64_t dims[3] = {(cuuint64_t)p.E, (cuuint64_t)p.T, (cuuint64_t)g->reserved};
    const cuuint64_t strides[2] = {(cuuint64_t)p.token_stride * 2, (cuuint64_t)p.block_stride * 2};  // bytes, dims 1..2
    const cuuint32_t box[3] = {(cuuint32_t)cols, (cuuint32_t)p.T, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<uint16_t*>(p.k), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return UCMX_EUNSUPPORTED;
    p.cs = cs;
    p.cg_per_item = cols / 8;
    int threads = ((cols / 2 + 31) / 32) * 32;
    const int grid = p.n * cs;
#define UCMX_TILE_CASE(M)                                                                              \
    case M: {                                                                                          \
        auto kern = pool_blocks_tile_kernel<M>;                                                        \
        UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<grid, threads, smem, st>>>(tmap, p);                                                    \
    } break;
    switch (mode) {
        UCMX_TILE_CASE(UCMX_POOL_MEAN)
        UCMX_TILE_CASE(UCMX_POOL_MAX)
        UCMX_TILE_CASE(UCMX_POOL_MIN)
        default:
            UCMX_TILE_CASE(UCMX_POOL_SUM)
    }
#undef UCMX_TILE_CASE
    UCMX_LAUNCH_CHECK("pool_blocks_tile_kernel");
    return UCMX_OK;
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_pool_blocks(const void* k_cache, const ucmx_kv_geometry* g, const int32_t* block_ids,
                                    const int32_t* out_slots, int64_t n_out_slots, int32_t n, int32_t mode, int32_t round_bf16,
                                    int32_t n_rep, int32_t rep_index, void* out_bf16, float* out_f32,
                                    ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n < 0) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (!k_cache || !g || !block_ids || (!out_bf16 && !out_f32)) return UCMX_EPARAM;
    if (g->reserved < 1 || n_out_slots < 1) {
        set_last_text("pool_blocks: the geometry must carry the number of blocks in the cache and the call the rows of the table");
        return UCMX_EPARAM;
    }
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
    p.cache_blocks = g->reserved;
    p.out_rows = n_out_slots;
    p.n = n;
    p.round_bf16 = round_bf16;
    p.n_rep = n_rep;
    p.rep_index = rep_index;
    p.out_bf16 = (uint16_t*)out_bf16;
    p.out_f32 = out_f32;
    p.err = error_word();
    {
        PoolParams pt = p;
        const int32_t rc = launch_pool_tile(pt, g, mode, (cudaStream_t)stream);
        if (rc != UCMX_EUNSUPPORTED) return rc;
    }
    // With few blocks (a decode step pools one new block per request) a block's rows are cut into
    // column pieces so that the work still covers the machine; each column is summed by one thread
    // in token order either way, so results do not depend on the split.
    const int sms = sm_count();
    int cs = 1;
    const int n_cg_row = p.E / 8;
    while ((int64_t)n * cs < 4 * (int64_t)sms && cs < 8 && n_cg_row % (cs * 2) == 0 && n_cg_row / (cs * 2) >= 16) cs *= 2;
    p.cs = cs;
    p.cg_per_item = n_cg_row / cs;
    const int64_t piece_bytes = (int64_t)p.cg_per_item * 16;
    p.rows_per_stage = (int32_t)(kStageBytes / piece_bytes);
    if (p.rows_per_stage > p.T) p.rows_per_stage = p.T;
    p.chunks_per_block = (p.T + p.rows_per_stage - 1) / p.rows_per_stage;
    p.dense = (g->token_stride == E64 && cs == 1) ? 1 : 0;
    p.err = error_word();

    const int n_cg = p.cg_per_item;
    int threads = ((n_cg + 31) / 32) * 32;
    int cgt = 1;
    while (threads > 256 && cgt < kMaxColGroupsPerThread) {
        cgt *= 2;
        threads = (((n_cg + cgt - 1) / cgt + 31) / 32) * 32;
    }
    if (threads > 1024) return UCMX_EUNSUPPORTED;
    // a CTA that owns a single work item needs no more stages than the item has chunks
    p.stages = kStages;
    if ((int64_t)n * cs <= (int64_t)sms * 3 && p.chunks_per_block < kStages) p.stages = p.chunks_per_block;
    const size_t smem = 128 + (size_t)p.stages * kStageBytes;
    int ctas_per_sm = (int)((size_t)(220 * 1024) / (smem + 1024));
    if (ctas_per_sm > 8) ctas_per_sm = 8;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = (int64_t)sms * ctas_per_sm;
    if (grid > (int64_t)n * cs) grid = (int64_t)n * cs;

    cudaStream_t st = (cudaStream_t)stream;
    switch (mode) {
        case UCMX_POOL_MEAN: return launch_pool<UCMX_POOL_MEAN>(p, threads, cgt, (int)grid, smem, st);
        case UCMX_POOL_MAX: return launch_pool<UCMX_POOL_MAX>(p, threads, cgt, (int)grid, smem, st);
        case UCMX_POOL_MIN: return launch_pool<UCMX_POOL_MIN>(p, threads, cgt, (int)grid, smem, st);
        default: return launch_pool<UCMX_POOL_SUM>(p, threads, cgt, (int)grid, smem, st);
    }
}

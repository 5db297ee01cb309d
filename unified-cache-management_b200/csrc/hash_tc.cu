// Stage 1b on the 5th-generation tensor cores: sign-hash codes as a bf16 GEMM with an exactness net.
//
// The projection x[128] . W[128x128] of every key vector is a real GEMM (M = all token-heads of all
// blocks, N = K = 128; about 120 flop per byte moved), so it belongs on tcgen05: 128-vector tiles of
// the paged cache are brought in by tiled TMA loads (128-byte swizzle, the layout the MMA unit reads),
// one elected thread issues eight tcgen05.mma (M128 N128 K16, bf16 in, fp32 accumulate in TMEM) per
// tile, and sets of four epilogue warps read the accumulator back with tcgen05.ld, take signs and pack bits.
// One thread block per SM: five tile buffers, four accumulators (all 512 TMEM columns), three epilogue sets
// that take the tiles in turn, three fixer warps (below; they also start the reload of a buffer they are done with)
// and one thread that issues every MMA.
//
// Codes must be bit-identical to the checker's definition - the sign of an fp32 fused-multiply-add
// chain over d = 0..127 - while the tensor core adds in its own order.  With S the exact sum, the chain
// is off by at most 128 * 2^-24 * sum|x_d w_d| = 2^-17 * sum|x_d w_d| (the standard bound for recursive
// summation), and sum|x_d w_d| <= |x| |w_j| (Cauchy-Schwarz).  The epilogue trusts the tensor-core sign
// only when |acc| > 2^-15 * |x| * max_j|w_j|, four times that bound: the two sums then agree in sign as
// long as the tensor core's own error stays under 3 * 2^-17 * sum|x_d w_d|, that is, as long as it keeps
// about 15 bits against the sum of magnitudes.  Measured on 805 million bits (Gaussian keys, two seeds,
// and keys with outlier channels), the two signs never differed until the margin was lowered to 2^-30,
// so the tensor core in fact keeps about 24.  The few remaining bits (about one in four thousand for
// Gaussian data) go to a fixer warp, which runs the exact chain from the tile still sitting in shared
// memory and patches the stored code.  A chain is 128 dependent multiply-adds: run by the epilogue
// warps themselves it cost a quarter of the kernel's time (plus as much again for pooling the work); on
// a warp of its own it overlaps with everything else.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace ucmx {
namespace {

constexpr int kTileM = 128;
constexpr int kDim = 128;
constexpr int kBits = 128;
constexpr int kStagesA = 5;                       // tile buffers of the one thread block an SM holds
constexpr int kAcc = 4;                           // accumulators in tensor memory (4 x 128 columns: all of it)
constexpr int kSets = 3;                          // epilogue warp sets; tile i of the thread block goes to set i % kSets
constexpr int kFixers = 3;                        // fixer warps (warps 0, 2 and 3); tile i goes to fixer i % kFixers
constexpr int kHalfBytes = kTileM * 128;          // one 64-element K half of a tile: 128 rows x 128 B
constexpr int kTileBytes = 2 * kHalfBytes;        // 32 KiB
constexpr int kFirstSetWarp = 4;                  // a multiple of four: warp w reads TMEM lanes 32 (w % 4) ...
constexpr int kThreads = 32 * (kFirstSetWarp + 4 * kSets);   // warps 0, 2, 3: exact-chain fixers (and reloads), warp 1: MMA issue and TMEM owner, warps 4-15: epilogue sets
constexpr float kTau = 1.0f / 32768.0f;           // 2^-15
constexpr int kFallbackSlots = 256;               // doubtful bits one warp pools per tile when the fixer's queue is full
constexpr int kFixSlots = 128;                    // code words with doubtful bits a fixer warp takes per tile (about 5 are typical)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
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

struct TcParams {
    const uint16_t* w;     // [128][128] bf16, row = d, column = bit
    uint8_t* out;
    int64_t n_vec;         // dense: number of vectors
    int64_t n_tiles;
    int32_t paged, H, T, head_major, tiles_per_block;
    int32_t h_shift, tok_per_tile;   // H is a power of two (it divides the 128 rows of a tile): log2 H, and 128 / H
    const int32_t* ids;
    const int32_t* out_slots;
    int64_t cache_blocks, out_rows;   // paged: blocks in the cache, rows of the code table
    int32_t* err;
};

// ---- PTX wrappers ------------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
                     "r"(smem_u32(dst)), "l"(m), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, int c0, int c1, int c2, int c3, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::
            "r"(smem_u32(dst)),
        "l"(m), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                               // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                               // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                               // layout type: SWIZZLE_128B
    return d;
}
// D fp32, A and B bf16, both K-major, N = 128, M = 128
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBits >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// sixteen accumulator columns of this thread's row, without waiting for them ...
__device__ __forceinline__ void tmem_ld16_start(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
// ... and the wait for everything started so far.  The registers are passed through the wait so that no use of them
// can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld16_wait(uint32_t (&v)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                   "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

// byte offset of element (row, k) inside a [128 x 128] bf16 K-major tile stored as two swizzled halves
__device__ __forceinline__ uint32_t sw_offset(int row, int k)
{
    const int half = k >> 6, c = (k & 63) >> 3;
    return (uint32_t)(half * kHalfBytes + row * 128 + ((c ^ (row & 7)) << 4) + ((k & 7) << 1));
}

struct alignas(16) Barriers {      // (what follows it in shared memory is accessed 16 bytes at a time)
    uint64_t full[kStagesA], acc_full[kAcc], acc_empty[kAcc], fix_ready[kStagesA];
    uint32_t tmem_base;
    int32_t abort_flag;
    uint32_t fix_n[kStagesA];   // code words queued for the fixer, per stage
};

__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity)   // one non-blocking poll
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// One thread starts the load of a tile: expect the bytes on the buffer's barrier, then the two halves of the tile.
// Paged: (cache block id, tile of the block) name the box; an id outside the cache reads outside the tensor map -
// TMA fills zeros and the tile's codes are not stored.  Dense: the first row.
__device__ __forceinline__ void start_tile_load(const CUtensorMap* tmap, unsigned char* dst, uint64_t* bar, bool paged, int id,
                                                int t0, int row0)
{
    mbar_expect_tx(bar, kTileBytes);
    if (paged) {
        tma_load_4d(dst, tmap, 0, 0, t0, id, bar);
        tma_load_4d(dst + kHalfBytes, tmap, 64, 0, t0, id, bar);
    } else {
        tma_load_2d(dst, tmap, 0, row0, bar);
        tma_load_2d(dst + kHalfBytes, tmap, 64, row0, bar);
    }
}

// PAGED: the vectors are key blocks of a paged cache named by a list (else: a dense array of vectors).  A template switch:
// the kernel stalls on instruction fetch more than on anything else, so it does not carry the other form's code.
template <bool PAGED>
__global__ void __launch_bounds__(kThreads, 1)
hash_encode_tc_kernel(const __grid_constant__ CUtensorMap tmap, TcParams p)
{
    extern __shared__ unsigned char smem_raw[];
    // rounded up to 1 KiB (the swizzle's period) by pointer arithmetic on the shared array, so that every pointer
    // derived from it is known to be a shared-memory pointer and its loads and stores are shared-memory instructions
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sA = smem;                                   // kStagesA tiles
    unsigned char* sB = smem + kStagesA * kTileBytes;            // W^T as the B operand: row = bit, K = d
    float* wnorm = reinterpret_cast<float*>(sB + kTileBytes);    // |w_j|
    Barriers* bars = reinterpret_cast<Barriers*>(wnorm + kBits);
    uint16_t* fb_list = reinterpret_cast<uint16_t*>(bars + 1);           // epilogue warps x kFallbackSlots
    uint8_t* fb_res = reinterpret_cast<uint8_t*>(fb_list + 4 * kSets * kFallbackSlots);
    uint32_t* wmax_bits = reinterpret_cast<uint32_t*>(fb_res + 4 * kSets * kFallbackSlots);   // max_j |w_j|
    uint4* fixq = reinterpret_cast<uint4*>(wmax_bits + 4);   // kStagesA x kFixSlots: {row | word index << 8, doubtful bits, word, -}

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- one-time set-up: barriers, the B operand (transposed and swizzled by hand), column norms, TMEM
    if (tid == 0) {
        for (int s = 0; s < kStagesA; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->fix_ready[s], 128);    // every epilogue thread has queued its doubtful words and stored the others
            bars->fix_n[s] = 0;
        }
        for (int a = 0; a < kAcc; ++a) {
            mbar_init(&bars->acc_full[a], 1);
            mbar_init(&bars->acc_empty[a], 128);
        }
        bars->abort_flag = 0;
        *wmax_bits = 0;
        mbar_init_fence();
    }
    __syncthreads();
    for (int i = tid; i < kDim * kBits / 8; i += kThreads) {
        const int d = i / (kBits / 8), j0 = (i - d * (kBits / 8)) * 8;   // eight bits j0..j0+7 of row d: W[d][j] -> B[row j][k d]
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.w) + i);
        const uint32_t e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 8; ++t)
            *reinterpret_cast<uint16_t*>(sB + sw_offset(j0 + t, d)) = (uint16_t)(e[t >> 1] >> ((t & 1) * 16));
    }
    __syncthreads();
    if (tid < kBits) {
        float s2 = 0.0f;
#pragma unroll 4
        for (int c = 0; c < 16; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(sB + sw_offset(tid, c * 8));
            const float e[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y), bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
#pragma unroll
            for (int t = 0; t < 8; ++t) s2 = fmaf(e[t], e[t], s2);
        }
        wnorm[tid] = sqrtf(s2) * 1.0001f;
        atomicMax(wmax_bits, __float_as_uint(wnorm[tid]));   // non-negative floats order like their bit patterns
    }
    fence_proxy_async();            // the hand-written B tile must be visible to the MMA unit
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(kAcc * kBits)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    // (tile numbers fit in 31 bits - the launch checks it - so everything below counts in 32 bits: the 64-bit
    // divisions and remainders of a tile counter by 5, 4 and the tiles of a block were a good part of each role's code)
    const int first = (int)blockIdx.x, stride = (int)gridDim.x;
    const int my_tiles = (int64_t)first < p.n_tiles ? (int)((p.n_tiles - first + stride - 1) / stride) : 0;

    if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issue (and the first loads), one thread
        // This thread is the kernel's serial resource - under load every one of its shared-memory operations (a
        // barrier poll, an MMA that reads its operands there) takes hundreds of cycles - so it does nothing but the
        // eight MMAs of a tile: it starts the loads of the first kStagesA tiles, and from then on the fixer warp that
        // is done with a tile's buffer starts the load of the tile that goes there next.
        const uint32_t b_addr = smem_u32(sB);
        for (int ld = 0; ld < my_tiles && ld < kStagesA; ++ld) {
            const int tile = first + ld * stride;
            int id = 0, t0 = 0;
            if (PAGED) {
                const uint32_t blk = (uint32_t)tile / (uint32_t)p.tiles_per_block;      // (tile numbers fit in 31 bits)
                id = __ldg(p.ids + blk);
                t0 = (int)((uint32_t)tile - blk * (uint32_t)p.tiles_per_block) * p.tok_per_tile;
            }
            start_tile_load(&tmap, sA + (size_t)ld * kTileBytes, &bars->full[ld], PAGED, id, t0, tile * kTileM);
        }
        int mm_s = 0, mm_a = 0;
        uint32_t full_par = 0, acc_par = 1, idle = 0;
        for (int mm = 0; mm < my_tiles;) {
            if (mbar_test(&bars->full[mm_s], full_par) && mbar_test(&bars->acc_empty[mm_a], acc_par)) {
                tc_fence_after();
                const uint32_t a_addr = smem_u32(sA + (size_t)mm_s * kTileBytes);
#pragma unroll
                for (int k = 0; k < kDim / 16; ++k) {
                    const uint32_t koff = (uint32_t)((k >> 2) * kHalfBytes + (k & 3) * 32);
                    umma_bf16(tmem_base + (uint32_t)mm_a * kBits, smem_desc_sw128(a_addr + koff), smem_desc_sw128(b_addr + koff),
                              k > 0 ? 1u : 0u);
                }
                umma_commit(&bars->acc_full[mm_a]);   // arrives when the eight MMAs above have completed
                ++mm;
                if (++mm_s == kStagesA) {
                    mm_s = 0;
                    full_par ^= 1u;
                }
                if (++mm_a == kAcc) {
                    mm_a = 0;
                    acc_par ^= 1u;
                }
                idle = 0;
            } else if (++idle > (1u << 24) || *(volatile int32_t*)&bars->abort_flag) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 1);
                break;
            }
        }
    } else if (warp == 0 || warp == 2 || warp == 3) {
        // ------------------------------------------------------------------ fixer: exact chains for the queued bits
        // The fp32 FMA chain over d, in order, from the tile and the weights in shared memory; one lane per
        // queued code word (usually one doubtful bit in it).  The lane settles the bits and stores the word.
        // The tile's buffer is held until the vectors are in registers; what does not depend on the queue
        // (where the tile's codes go) is worked out while waiting.
        for (int it = (warp + 1) >> 1; it < my_tiles; it += kFixers) {     // warps 0, 2, 3 -> fixers 0, 1, 2
            const int s = it % kStagesA;
            const uint32_t par = (uint32_t)((it / kStagesA) & 1);
            const int tile = first + it * stride;
            int64_t blk = 0, slot = 0;
            int sub = 0, id = 0;
            if (PAGED) {
                blk = (int64_t)((uint32_t)tile / (uint32_t)p.tiles_per_block);
                sub = (int)((uint32_t)tile - (uint32_t)blk * (uint32_t)p.tiles_per_block);
                id = checked_block_id(p.ids, blk, p.cache_blocks, nullptr);
                slot = id < 0 ? -1 : checked_out_row(p.out_slots, blk, p.out_rows, nullptr);
            }
            // the tile that goes into this buffer next (kStagesA tiles on): lane 0 starts its load as soon as this
            // tile's vectors are in registers; what it needs for that is asked for now, ahead of the waits
            const int nt = it + kStagesA;
            int n_id = 0, n_t0 = 0;
            const int n_tile = first + nt * stride;
            if (PAGED && nt < my_tiles) {
                const uint32_t nblk = (uint32_t)n_tile / (uint32_t)p.tiles_per_block;
                n_id = __ldg(p.ids + nblk);
                n_t0 = (int)((uint32_t)n_tile - nblk * (uint32_t)p.tiles_per_block) * p.tok_per_tile;
            }
            // First the tile's landing, then its epilogue.  The order matters: a parity wait is only right for a
            // barrier that is at most one phase behind, and this warp may come here while the buffer's previous
            // tile (another fixer's) is still in its epilogue; the landing of this tile, however, comes after that.
            if (!mbar_wait(&bars->full[s], par) || !mbar_wait(&bars->fix_ready[s], par)) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 1);
                break;
            }
            if (*(volatile int32_t*)&bars->abort_flag) break;
            const int n = (int)min(*(volatile uint32_t*)&bars->fix_n[s], (uint32_t)kFixSlots);
            const unsigned char* xa = sA + (size_t)s * kTileBytes;
            const uint4* q = fixq + s * kFixSlots;
            // Passes of 32 queued words.  Once the vectors of the last pass are in registers nothing here needs
            // the tile any more (the weights stay in shared memory), so the stage is released before the chains run.
            const int passes = (n + 31) >> 5;
            if (passes == 0) {
                __syncwarp();                                  // every lane has read the count before it is reset
                if (lane == 0) {
                    bars->fix_n[s] = 0;
                    if (nt < my_tiles)
                        start_tile_load(&tmap, sA + (size_t)s * kTileBytes, &bars->full[s], PAGED, n_id, n_t0, n_tile * kTileM);
                }
            }
            for (int ps = 0; ps < passes; ++ps) {
                const int e = ps * 32 + lane;
                const uint4 ent = e < n ? q[e] : make_uint4(0xffffffffu, 0u, 0u, 0u);   // x = ~0: nothing here
                const bool live = ent.x != 0xffffffffu;
                const int row = (int)(ent.x & 127u), cw = (int)((ent.x >> 8) & 3u);
                uint4 xv[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) xv[c] = *reinterpret_cast<const uint4*>(xa + sw_offset(row, c * 8));
                if (ps == passes - 1) {
                    // The loads must have delivered before the stage goes.  Only an instruction that reads the
                    // registers makes a lane wait for them, so every lane folds its vector into one word and the
                    // warp votes on it (the vote is also the point where the lanes meet).
                    uint32_t fold = 0;
#pragma unroll
                    for (int c = 0; c < 16; ++c) fold ^= xv[c].x ^ xv[c].y ^ xv[c].z ^ xv[c].w;
                    const unsigned seen = __ballot_sync(0xffffffffu, fold != 0x9e3779b9u);
                    if (lane == 0 && seen != 0xdeadbeefu) {
                        bars->fix_n[s] = 0;
                        if (nt < my_tiles)                      // the buffer is free: the tile that goes there next
                            start_tile_load(&tmap, sA + (size_t)s * kTileBytes, &bars->full[s], PAGED, n_id, n_t0, n_tile * kTileM);
                    }
                }
                if (!live) continue;
                uint32_t word = ent.z, pend = ent.y;
                while (pend) {
                    const int j = __ffs(pend) - 1;
                    pend &= pend - 1;
                    const int col = cw * 32 + j;
                    float acc = 0.0f;
                    // (the vector stays packed: without this the compiler widens all 128 values to fp32 ahead of the
                    // loop over the doubtful bits and spills half of them)
#pragma unroll
                    for (int c = 0; c < 16; c += 4)
                        asm volatile("" : "+r"(xv[c].x), "+r"(xv[c].y), "+r"(xv[c].z), "+r"(xv[c].w), "+r"(xv[c + 1].x), "+r"(xv[c + 1].y),
                                          "+r"(xv[c + 1].z), "+r"(xv[c + 1].w), "+r"(xv[c + 2].x), "+r"(xv[c + 2].y), "+r"(xv[c + 2].z),
                                          "+r"(xv[c + 2].w), "+r"(xv[c + 3].x), "+r"(xv[c + 3].y), "+r"(xv[c + 3].z), "+r"(xv[c + 3].w));
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(sB + sw_offset(col, c * 8));
                        acc = fmaf(bf16lo(xv[c].x), bf16lo(wv.x), acc);
                        acc = fmaf(bf16hi(xv[c].x), bf16hi(wv.x), acc);
                        acc = fmaf(bf16lo(xv[c].y), bf16lo(wv.y), acc);
                        acc = fmaf(bf16hi(xv[c].y), bf16hi(wv.y), acc);
                        acc = fmaf(bf16lo(xv[c].z), bf16lo(wv.z), acc);
                        acc = fmaf(bf16hi(xv[c].z), bf16hi(wv.z), acc);
                        acc = fmaf(bf16lo(xv[c].w), bf16lo(wv.w), acc);
                        acc = fmaf(bf16hi(xv[c].w), bf16hi(wv.w), acc);
                    }
                    word = (word & ~(1u << j)) | ((acc > 0.0f ? 1u : 0u) << j);
                }
                int64_t orow;
                if (PAGED) {
                    const int t = sub * p.tok_per_tile + (row >> p.h_shift), h = row & (p.H - 1);
                    orow = (id < 0 || slot < 0) ? -1 : p.head_major ? (slot * p.H + h) * p.T + t : (slot * p.T + t) * p.H + h;
                } else {
                    const int64_t v = (int64_t)tile * kTileM + row;
                    orow = v < p.n_vec ? v : -1;
                }
                if (orow >= 0) reinterpret_cast<uint32_t*>(p.out + orow * 16)[cw] = word;
            }
        }
    } else if (warp >= kFirstSetWarp) {
        // ------------------------------------------------------------------ epilogue: signs, margin test, exact fallback
        const int q = warp & 3;                  // the TMEM lane quarter this warp may read
        const int m = q * 32 + lane;             // tile row = vector
        // Paged: which list entry and which tile of its block a tile is, advanced without divisions; the entry's cache
        // block and code-table row group are asked for one tile ahead, so the stores at the end of a tile never wait.
        const int set = (warp - kFirstSetWarp) >> 2;
        int tok = 0, h = 0, blk = 0, sub = 0, step_blk = 0, step_sub = 0, nxt_id = 0, nxt_slot = 0;
        if (PAGED) {
            tok = m >> p.h_shift;
            h = m - tok * p.H;
            const int mine0 = first + set * stride, step = kSets * stride;   // this set's first tile, and its stride
            blk = mine0 / p.tiles_per_block;
            sub = mine0 - blk * p.tiles_per_block;
            step_blk = step / p.tiles_per_block;
            step_sub = step - step_blk * p.tiles_per_block;
            if (set < my_tiles) {
                nxt_id = __ldg(p.ids + blk);
                nxt_slot = p.out_slots ? __ldg(p.out_slots + blk) : blk;
            }
        }
        for (int it = set; it < my_tiles; it += kSets) {
            const int s = it % kStagesA, a = it % kAcc;
            int64_t orow;                         // where this row's code goes (-1: nowhere)
            if (PAGED) {
                int id = nxt_id;
                int64_t slot = nxt_slot;
                if (id >= 0 && (int64_t)id >= p.cache_blocks) {
                    if (p.err) atomicExch(p.err, 3);
                    id = -1;
                }
                if (slot >= 0 && slot >= p.out_rows) {
                    if (p.err) atomicExch(p.err, 3);
                    slot = -1;
                }
                const int tk = sub * p.tok_per_tile + tok;
                orow = (id < 0 || slot < 0) ? -1 : p.head_major ? (slot * p.H + h) * p.T + tk : (slot * p.T + tk) * p.H + h;
                sub += step_sub;
                blk += step_blk;
                if (sub >= p.tiles_per_block) {
                    sub -= p.tiles_per_block;
                    ++blk;
                }
                if (it + kSets < my_tiles) {
                    nxt_id = __ldg(p.ids + blk);
                    nxt_slot = p.out_slots ? __ldg(p.out_slots + blk) : blk;
                }
            } else {
                const int64_t v = (int64_t)(first + it * stride) * kTileM + m;
                orow = v < p.n_vec ? v : -1;
            }
            if (!mbar_wait(&bars->acc_full[a], (uint32_t)((it / kAcc) & 1))) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 1);
                break;
            }
            if (*(volatile int32_t*)&bars->abort_flag) break;
            tc_fence_after();
            (void)mbar_wait(&bars->full[s], (uint32_t)((it / kStagesA) & 1));  // already complete: acquires the TMA-written tile
            const unsigned char* xa = sA + (size_t)s * kTileBytes;
            // An upper bound on |x|^2 of this row, cheaply: packed bf16 multiply-adds into eight pairs of
            // partial sums of eight terms each (a bf16 running sum of k non-negative terms is low by at
            // most k * 2^-8 relative, covered by the 1.05 below), added up in fp32.
            float x2 = 0.0f;
            {
                __nv_bfloat162 part[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) part[g] = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xa + sw_offset(m, c * 8));
                    const uint32_t e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&e[i]);
                        part[(c * 4 + i) & 7] = __hfma2(h, h, part[(c * 4 + i) & 7]);
                    }
                }
#pragma unroll
                for (int g = 0; g < 8; ++g) x2 += __low2float(part[g]) + __high2float(part[g]);
            }
            // one threshold for the whole row: |acc| <= tau |x| max_j|w_j| (a little wider than per column, no table look-up)
            // a row so small that its squares underflow in bf16 gets no trusted bits at all (threshold = infinity)
            // - unless every element is zero, as in the unwritten part of a block: the chain of such a row ends at +0
            // whatever the weights, so all of its bits are 0 and nothing is doubtful
            float thr;
            uint32_t keep = 0xffffffffu;
            if (x2 >= 1e-30f) {
                thr = kTau * sqrtf(x2 * 1.05f) * 1.0001f * __uint_as_float(*wmax_bits);
            } else {
                uint32_t any = 0;
#pragma unroll 4
                for (int c = 0; c < 16; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xa + sw_offset(m, c * 8));
                    any |= (v.x | v.y | v.z | v.w) & 0x7fff7fffu;
                }
                thr = any ? INFINITY : -1.0f;
                keep = any ? 0xffffffffu : 0u;
            }
            // The accumulator comes in eight pieces of sixteen columns, the next one on its way while the signs and
            // margins of the one at hand are worked out (what a warp waits for here is the round trip to tensor
            // memory, not the arithmetic).
            // Sign bits: shift each accumulator's sign into a word, highest column first (one funnel shift per value).
            // A set sign bit means "not positive"; an exact zero has a clear sign bit but is below any threshold, so
            // it is settled by the exact chain like every doubtful bit.  Then the smallest magnitude of each group
            // of eight columns (one min per value): only groups that dip under the threshold are looked at column
            // by column.
            uint32_t code[4], doubt[4];
            {
                // One code word (two pieces) per pass of a loop that is NOT unrolled: the kernel's instruction stream
                // is large, sixteen warps of three kinds share the instruction caches, and instruction fetch was the
                // most frequent stall; four copies of this body added 9 KB to it.
                uint32_t v[2][16];
                const uint32_t acc_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kBits);
                tmem_ld16_start(acc_addr + 7 * 16, v[1]);       // pieces are taken from the highest column down
#pragma unroll 1
                for (int pp = 3; pp >= 0; --pp) {
                    uint32_t neg = 0, unsure = 0;
#pragma unroll
                    for (int half = 1; half >= 0; --half) {
                        uint32_t (&cur)[16] = v[half];
                        tmem_ld16_wait(cur);
                        if (half == 1) tmem_ld16_start(acc_addr + (uint32_t)(pp * 2) * 16, v[0]);
                        else if (pp > 0) tmem_ld16_start(acc_addr + (uint32_t)(pp * 2 - 1) * 16, v[1]);
#pragma unroll
                        for (int j = 15; j >= 0; --j) neg = __funnelshift_l(cur[j], neg, 1);
#pragma unroll
                        for (int g8 = 0; g8 < 2; ++g8) {
                            float mn = fabsf(__uint_as_float(cur[g8 * 8]));
#pragma unroll
                            for (int j = 1; j < 8; ++j) mn = fminf(mn, fabsf(__uint_as_float(cur[g8 * 8 + j])));
                            if (mn <= thr) {
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    unsure |= (fabsf(__uint_as_float(cur[g8 * 8 + j])) <= thr ? 1u : 0u) << (half * 16 + g8 * 8 + j);
                            }
                        }
                    }
                    const uint32_t word = ~neg & keep;          // (selects, not an indexed store: the arrays stay in registers)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (k == pp) {
                            code[k] = word;
                            doubt[k] = unsure;
                        }
                }
            }
            // the accumulator is read: hand it back to the MMA warp
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[a]);
            // Exact recomputation of the doubtful bits: the fp32 FMA chain over d, in order.  The chain
            // of one bit cannot be split, but different bits can go to different lanes: the warp pools
            // its (row, column) pairs in shared memory and deals them out, so a tile with a handful of
            // doubtful bits costs one chain's latency instead of one per bit of the unluckiest lane.
            // A 32-bit word of the code that holds doubtful bits is not stored here: it goes, with the mask of
            // those bits, to the fixer, which stores it once they are settled.  Every word thus has one writer.
            bool queued = false;
            {
                const int wmine = (doubt[0] != 0) + (doubt[1] != 0) + (doubt[2] != 0) + (doubt[3] != 0);
                int wincl = wmine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, wincl, o);
                    if (lane >= o) wincl += v;
                }
                const int wtotal = __shfl_sync(0xffffffffu, wincl, 31);
                if (wtotal > 0) {
                    // one reservation per warp in the stage's queue
                    uint32_t base = 0;
                    if (lane == 0) base = atomicAdd(&bars->fix_n[s], (uint32_t)wtotal);
                    base = __shfl_sync(0xffffffffu, base, 0);
                    uint4* q = fixq + s * kFixSlots;
                    if (base + (uint32_t)wtotal > (uint32_t)kFixSlots) {
                        // no room: what the reservation covers below the capacity is marked empty and this warp
                        // settles its bits itself (below)
                        for (uint32_t e = base + (uint32_t)lane; e < (uint32_t)kFixSlots; e += 32) q[e] = make_uint4(0xffffffffu, 0u, 0u, 0u);
                    } else {
                        queued = true;
                        uint32_t pos = base + (uint32_t)(wincl - wmine);
#pragma unroll
                        for (int cw = 0; cw < 4; ++cw)
                            if (doubt[cw]) q[pos++] = make_uint4((uint32_t)m | ((uint32_t)cw << 8), doubt[cw], code[cw], 0u);
                    }
                }
            }
            if (!queued) {
                const int mine = __popc(doubt[0]) + __popc(doubt[1]) + __popc(doubt[2]) + __popc(doubt[3]);
                int incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                const int total = __shfl_sync(0xffffffffu, incl, 31);
                if (total > 0) {
                    uint16_t* list = fb_list + (warp - kFirstSetWarp) * kFallbackSlots;
                    uint8_t* res = fb_res + (warp - kFirstSetWarp) * kFallbackSlots;
                    int pos = incl - mine;
#pragma unroll
                    for (int cw = 0; cw < 4; ++cw) {
                        uint32_t pend = doubt[cw];
                        while (pend) {
                            const int j = __ffs(pend) - 1;
                            pend &= pend - 1;
                            if (pos < kFallbackSlots) list[pos] = (uint16_t)((m << 7) | (cw * 32 + j));
                            ++pos;
                        }
                    }
                    __syncwarp();
                    const int pooled = min(total, kFallbackSlots);
                    for (int e = lane; e < pooled; e += 32) {
                        const int row = list[e] >> 7, col = list[e] & 127;
                        float acc = 0.0f;
#pragma unroll 4
                        for (int c = 0; c < 16; ++c) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(xa + sw_offset(row, c * 8));
                            const uint4 wv = *reinterpret_cast<const uint4*>(sB + sw_offset(col, c * 8));
                            acc = fmaf(bf16lo(xv.x), bf16lo(wv.x), acc);
                            acc = fmaf(bf16hi(xv.x), bf16hi(wv.x), acc);
                            acc = fmaf(bf16lo(xv.y), bf16lo(wv.y), acc);
                            acc = fmaf(bf16hi(xv.y), bf16hi(wv.y), acc);
                            acc = fmaf(bf16lo(xv.z), bf16lo(wv.z), acc);
                            acc = fmaf(bf16hi(xv.z), bf16hi(wv.z), acc);
                            acc = fmaf(bf16lo(xv.w), bf16lo(wv.w), acc);
                            acc = fmaf(bf16hi(xv.w), bf16hi(wv.w), acc);
                        }
                        res[e] = acc > 0.0f ? 1 : 0;
                    }
                    __syncwarp();
                    pos = incl - mine;
#pragma unroll
                    for (int cw = 0; cw < 4; ++cw) {
                        uint32_t pend = doubt[cw];
                        while (pend) {
                            const int j = __ffs(pend) - 1;
                            pend &= pend - 1;
                            uint32_t bit;
                            if (pos < kFallbackSlots) {
                                bit = res[pos];
                            } else {
                                // more doubtful bits than the pool holds (degenerate inputs): the owner does its own
                                const int col = cw * 32 + j;
                                float acc = 0.0f;
                                for (int d = 0; d < kDim; ++d) {
                                    const float xv = __uint_as_float((uint32_t)*reinterpret_cast<const uint16_t*>(xa + sw_offset(m, d)) << 16);
                                    const float wv = __uint_as_float((uint32_t)*reinterpret_cast<const uint16_t*>(sB + sw_offset(col, d)) << 16);
                                    acc = fmaf(xv, wv, acc);
                                }
                                bit = acc > 0.0f ? 1u : 0u;
                            }
                            ++pos;
                            code[cw] = (code[cw] & ~(1u << j)) | (bit << j);
                        }
                    }
                    __syncwarp();
                }
            }
            // store the code, then tell the fixer, which releases the stage when it has what it needs of the tile
            // (a word the fixer still has to settle is stored as it stands; the fixer's store comes after the barrier
            // below and therefore after this one)
            if (orow >= 0) *reinterpret_cast<uint4*>(p.out + orow * 16) = make_uint4(code[0], code[1], code[2], code[3]);
            mbar_arrive(&bars->fix_ready[s]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAcc * kBits) : "memory");
    }
}

}  // namespace

// Returns UCMX_EUNSUPPORTED when the tensor-core path does not apply; the caller then runs the
// CUDA-core kernel, which produces the same codes.
int32_t hash_encode_tc(const void* x, int64_t n_vec, int64_t x_stride, const ucmx_kv_geometry* g, const int32_t* ids,
                       const int32_t* out_slots, int64_t n_out_rows, int32_t n_blocks, const void* w, int32_t dim,
                       int32_t bits, int32_t head_major, uint8_t* out, cudaStream_t st)
{
    EncodeTiledFn enc = encode_fn();
    if (!enc || dim != kDim || bits != kBits || ((uintptr_t)out & 15) || ((uintptr_t)x & 15)) return UCMX_EUNSUPPORTED;
    TcParams p{};
    p.w = (const uint16_t*)w;
    p.out = out;
    p.err = error_word();
    alignas(64) CUtensorMap tmap;
    CUresult r;
    if (g) {
        const int H = g->n_kv_heads, T = g->block_tokens;
        if (g->head_dim != kDim || g->reserved <= 0 || H < 1 || H > kTileM || kTileM % H || T % (kTileM / H)) return UCMX_EUNSUPPORTED;
        if (kTileM / H > 256 || (g->token_stride % 8) || (g->block_stride % 8)) return UCMX_EUNSUPPORTED;
        const cuuint64_t dims[4] = {(cuuint64_t)kDim, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)g->reserved};
        const cuuint64_t strides[3] = {(cuuint64_t)kDim * 2, (cuuint64_t)g->token_stride * 2, (cuuint64_t)g->block_stride * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)H, (cuuint32_t)(kTileM / H), 1};
        const cuuint32_t es[4] = {1, 1, 1, 1};
        r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        p.paged = 1;
        p.H = H;
        p.T = T;
        p.head_major = head_major;
        p.tiles_per_block = T * H / kTileM;
        p.tok_per_tile = kTileM / H;
        for (p.h_shift = 0; (1 << p.h_shift) < H; ++p.h_shift) {}
        p.ids = ids;
        p.out_slots = out_slots;
        p.cache_blocks = g->reserved;
        p.out_rows = n_out_rows;
        p.n_tiles = (int64_t)n_blocks * p.tiles_per_block;
        if (p.n_tiles > 0x7fffffffll) return UCMX_EUNSUPPORTED;
    } else {
        if (x_stride % 8 || n_vec < 1 || n_vec > 0x7fffffffll) return UCMX_EUNSUPPORTED;
        const cuuint64_t dims[2] = {(cuuint64_t)kDim, (cuuint64_t)n_vec};
        const cuuint64_t strides[1] = {(cuuint64_t)x_stride * 2};
        const cuuint32_t box[2] = {64, kTileM};
        const cuuint32_t es[2] = {1, 1};
        r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        p.n_vec = n_vec;
        p.n_tiles = (n_vec + kTileM - 1) / kTileM;
    }
    if (r != CUDA_SUCCESS) return UCMX_EUNSUPPORTED;
    const size_t smem = 1024 + (size_t)kStagesA * kTileBytes + kTileBytes + kBits * sizeof(float) + sizeof(Barriers) + 4 * kSets * kFallbackSlots * 3 + 16 + (size_t)kStagesA * kFixSlots * 16 + 128;
    UCMX_CUDA(cudaFuncSetAttribute(hash_encode_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    UCMX_CUDA(cudaFuncSetAttribute(hash_encode_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid = (int64_t)sm_count();
    if (grid > p.n_tiles) grid = p.n_tiles;
    if (p.paged) hash_encode_tc_kernel<true><<<(unsigned)grid, kThreads, smem, st>>>(tmap, p);
    else hash_encode_tc_kernel<false><<<(unsigned)grid, kThreads, smem, st>>>(tmap, p);
    UCMX_LAUNCH_CHECK("hash_encode_tc_kernel");
    return UCMX_OK;
}

}  // namespace ucmx

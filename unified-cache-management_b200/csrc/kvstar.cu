// KVStar multi-query softmax-vote retrieval: every query row of a request (x recent tokens x Hq heads)
// is dotted with the representations of its KV head at all S = n_blocks*M positions, softmaxed over
// S, and each block collects the probability mass of its M positions over all rows; the blocks with
// the most votes are kept (the reference's CPU kernel: KVStar::Execute,
// ucm/sparse/kvstar/retrieve/core/domain/retrieve_task/simd_compute_kernel.cpp:635-764; its caller
// ucm/sparse/kvstar/multistep.py:240-262; block representations multistep.py:279-316).
//
// This is the one scoring variant that is a real GEMM (x*Hq rows against S columns, half precision),
// so the dot products run on tcgen05.  The softmax needs the maximum and the sum over all S, which
// no single CTA sees; it is therefore split:
//   pass 1 (one tile = one block of M positions): per query row, the block-local maximum m (kept in
//           units of log2, m = max * log2 e) and p = sum_s 2^(score_s * log2 e - m), 8 bytes per
//           (block, row) instead of M scores;
//   pass 2a (per request and row): the global maximum and normaliser from the (m, p) pairs;
//   pass 2b (per block): votes = sum_rows p * 2^(m - m_row) / Z_row.
// The representations are read exactly once; the (m, p) pairs add about 6 % traffic.
//
// Tensor-core mapping of pass 1: accumulator rows (TMEM lanes) are query rows and columns are the M
// positions of the block, so the reductions over positions are private to a thread.  A KV head has only
// x*g query rows (32 for 8 tokens of a 4-way group) but the instruction wants 128, so several heads
// share one instruction through a block-diagonal A operand: row (head, query) holds its query in the
// K range of its own head and zeros elsewhere, and the B operand is simply the block's [M positions] x
// [heads x d_pruned] slab as it lies in memory, brought in by tiled TMA loads with the 128-byte swizzle.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace ucmx {
namespace {

constexpr int kRows = 128;              // accumulator rows per instruction (TMEM lanes)
constexpr int kChunkA = kRows * 128;    // one 64-element K chunk of the A operand: 128 rows x 128 B
constexpr int kTcThreads = 320;         // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5 and 6-9: two epilogue sets
constexpr float kLog2e = 1.4426950408889634f;

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

struct KsParams {
    const uint16_t* q;          // half [sum x][Hq][d_orig]
    const int32_t* q_offsets;   // [n_req+1] first query token row of each request
    const int64_t* pruned;      // [n_req][H][dp] channel of d_orig behind each kept channel, or NULL
    const uint16_t* reps;       // half [n_slots][M][H][dp]
    const int32_t* offsets;     // [n_req+1] candidate blocks of each request
    const int32_t* slot_ids;    // [total] table slot of each candidate, or NULL = identity
    int32_t n_slots;            // rows of the table (the tensor-core kernels read through a tensor map of that extent,
                                // so a slot beyond it reads zeros there; the CUDA-core kernel checks it)
    float2* part;               // [total][Rtot] (m, p)
    float2* stats;              // [n_req][Rtot] (m_row, 1/Z_row)
    float* out;                 // [total] votes
    int32_t* err;
    int32_t n_req, total, M, H, dp, C, Hq, gq, d_orig;
    int32_t Rp, Rtot;           // padded query rows per KV head, H*Rp
    int32_t hpg, G, cpg;        // heads per MMA group, groups, 64-element K chunks per group
    uint32_t idesc;
    int32_t stages, tile_bytes;
    int32_t n_acc;              // accumulator sets in tensor memory (2 or 4)
};

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ------------------------------------------------------------------------------------ PTX wrappers

// The representations are read once: evict-first, so that the gigabyte passing through L2 does not push out the
// 74 MB of (maximum, sum) pairs this pass writes and the two small kernels after it read.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, int x, int y, uint64_t* bar)
{
    const uint64_t pol = l2_evict_first_policy();
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::
            "r"(smem_u32(dst)),
        "l"(m), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol)
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
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// tcgen05.ld split into issue and wait, so that one load can be in flight while the previous one is
// consumed.  The wait names the registers as read-write operands: nothing that uses them may be
// scheduled before it.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                   "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]),
                   "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]),
                   "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :
                 : "memory");
}

// 64 consecutive columns of this warp's 32 lanes, valid on return
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&v)[64])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,"
        "%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]),
          "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]),
          "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]),
          "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]),
          "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
        : "r"(taddr)
        : "memory");
}

// One MMA of the fully specialised issue sequence (64 positions per block, 64-element K chunks):
// operand offsets are immediates, so each instruction costs three integer adds.
template <int I, int CPG, int POS = 64>   // POS: positions (B rows, accumulator columns) per instruction
__device__ __forceinline__ void umma_f16_step(uint32_t d_base, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc)
{
    constexpr int c = I >> 2, k4 = I & 3, g = c / CPG, kc = c % CPG;
    constexpr int a_off = (c * kChunkA + k4 * 32) >> 4, b_off = (c * POS * 128 + k4 * 32) >> 4, d_off = g * POS;
    constexpr int acc = (kc | k4) ? 1 : 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 ta, tb, td;\n\t.reg .b64 da, db;\n\t"
        "add.u32 ta, %1, %5;\n\t"
        "add.u32 tb, %2, %6;\n\t"
        "add.u32 td, %0, %7;\n\t"
        "mov.b64 da, {ta, %3};\n\t"
        "mov.b64 db, {tb, %3};\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [td], da, db, %4, p;\n\t}" ::"r"(d_base),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(a_off), "n"(b_off), "n"(d_off), "n"(acc)
        : "memory");
}
template <int CPG, int POS = 64>
__device__ __forceinline__ void umma_f16_block16(uint32_t d_base, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc)
{
    umma_f16_step<0, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<1, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<2, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<3, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<4, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<5, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<6, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<7, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<8, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<9, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<10, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<11, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<12, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<13, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<14, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
    umma_f16_step<15, CPG, POS>(d_base, a_lo, b_lo, desc_hi, idesc);
}

struct alignas(8) KsBarriers {
    uint64_t full[8], empty[8], acc_full[4], acc_empty[4], a_ready;
    uint32_t tmem_base;
    int32_t abort_flag;
};

// Block-diagonal A operand of one request: accumulator row r = (local head r / Rp, query row r % Rp);
// its 16-byte units inside the K range of its own head hold the query (through the channel list when
// dimensions were pruned), every other unit is zero.  Called by 128 threads, one row each.
__device__ void build_a_operand(unsigned char* sA, const KsParams& p, int req, int row)
{
    const int hl = row / p.Rp, j = row - hl * p.Rp;
    const int xq = j / p.gq, gg = j - xq * p.gq;
    const int q0 = __ldg(p.q_offsets + req), nx = __ldg(p.q_offsets + req + 1) - q0;
    const bool live = hl < p.hpg && xq < nx;
    for (int g = 0; g < p.G; ++g) {
        const int h = g * p.hpg + hl;
        const uint16_t* qrow = p.q + ((int64_t)(q0 + xq) * p.Hq + (h * p.gq + gg)) * p.d_orig;
        const int64_t* pr = p.pruned ? p.pruned + ((int64_t)req * p.H + h) * p.dp : nullptr;
        for (int kc = 0; kc < p.cpg; ++kc) {
            unsigned char* chunk = sA + (size_t)(g * p.cpg + kc) * kChunkA + row * 128;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int col = kc * 64 + u * 8;            // first K column of this unit inside the group
                uint4 val = make_uint4(0, 0, 0, 0);
                if (live && col / p.dp == hl) {
                    const int d0 = col - hl * p.dp;
                    uint16_t e[8];
                    if (pr) {
#pragma unroll
                        for (int t = 0; t < 8; ++t) e[t] = __ldg(qrow + __ldg(pr + d0 + t));
                    } else {
                        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qrow + d0));
                        *reinterpret_cast<uint4*>(e) = raw;
                    }
                    val.x = e[0] | ((uint32_t)e[1] << 16);
                    val.y = e[2] | ((uint32_t)e[3] << 16);
                    val.z = e[4] | ((uint32_t)e[5] << 16);
                    val.w = e[6] | ((uint32_t)e[7] << 16);
                }
                *reinterpret_cast<uint4*>(chunk + ((u ^ (row & 7)) << 4)) = val;
            }
        }
    }
}

// ------------------------------------------------------------------------------ pass 1, tensor cores
template <int NM>   // 64-element K chunks per head group (1 or 2) of the specialised shape: 64 positions per block and
                    // heads * d_pruned == 256, whose 16 instructions per block are issued with immediate offsets; else 0
__global__ void __launch_bounds__(kTcThreads, 1)
kvstar_partial_tc_kernel(const __grid_constant__ CUtensorMap tmap, KsParams p)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    unsigned char* sA = smem;                                            // G*cpg chunks of 16 KiB
    unsigned char* sB = sA + (size_t)p.G * p.cpg * kChunkA;              // stages of tile_bytes
    KsBarriers* bars = reinterpret_cast<KsBarriers*>(sB + (size_t)p.stages * p.tile_bytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // contiguous run of candidate blocks per CTA, so that the A operand changes as rarely as possible
    const int t0 = (int)((int64_t)p.total * blockIdx.x / gridDim.x);
    const int t1 = (int)((int64_t)p.total * (blockIdx.x + 1) / gridDim.x);
    const int my_tiles = t1 - t0;
    const int acc_cols = p.G * p.M;                                      // TMEM columns of one accumulator set
    const int want_cols = acc_cols * p.n_acc;
    const uint32_t tmem_cols = want_cols <= 32 ? 32u : want_cols <= 64 ? 64u : want_cols <= 128 ? 128u : want_cols <= 256 ? 256u : 512u;

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        for (int a = 0; a < 4; ++a) {
            mbar_init(&bars->acc_full[a], 1);
            mbar_init(&bars->acc_empty[a], 128);
        }
        mbar_init(&bars->a_ready, 128);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (my_tiles > 0 && tid < kRows) build_a_operand(sA, p, find_request(p.offsets, p.n_req, t0), tid);
    fence_proxy_async();            // the hand-written A operand must be visible to the MMA unit
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const int n_chunks = p.G * p.cpg;
    const int chunk_b = p.M * 128;                                       // bytes of one K chunk of a tile

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------------ TMA producer
        int s = 0;
        uint32_t par = 0;
        int slot_next = my_tiles > 0 ? (p.slot_ids ? __ldg(p.slot_ids + t0) : t0) : 0;
        for (int it = 0; it < my_tiles; ++it, s = (s + 1 == p.stages ? 0 : s + 1), par ^= (s == 0 ? 1u : 0u)) {
            const int slot = slot_next;
            if (it + 1 < my_tiles) slot_next = p.slot_ids ? __ldg(p.slot_ids + t0 + it + 1) : t0 + it + 1;   // in flight during the wait
            if (!mbar_wait(&bars->empty[s], par ^ 1u)) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 5);
                break;
            }
            if (*(volatile int32_t*)&bars->abort_flag) break;
            unsigned char* dst = sB + (size_t)s * p.tile_bytes;
            mbar_expect_tx(&bars->full[s], (uint32_t)p.tile_bytes);
            // a negative slot reads outside the tensor: TMA fills zeros, the epilogue marks the block empty
            for (int c = 0; c < n_chunks; ++c) tma_load_2d(dst + (size_t)c * chunk_b, &tmap, c * 64, slot * p.M, &bars->full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        // One thread issues every instruction, and an M128 N64 K16 instruction occupies the tensor core for
        // far less time than a lone thread needs for a few dozen dependent instructions; whatever this
        // loop executes between two MMAs is therefore tensor-core idle time.  For the common shape the
        // sixteen instructions of a block are issued from immediates (umma_f16_block16), stage and
        // accumulator indices are counters, and there is a single commit per block.
        const uint32_t a_addr = smem_u32(sA);
        int req = my_tiles > 0 ? find_request(p.offsets, p.n_req, t0) : 0;
        int req_end = my_tiles > 0 ? __ldg(p.offsets + req + 1) : 0;
        uint32_t a_gen = 0;
        const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(0) >> 32);
        const uint32_t a_lo = (uint32_t)smem_desc_sw128(a_addr);
        const uint32_t idesc = p.idesc;
        const int stages = p.stages, n_acc = p.n_acc, tile_bytes = p.tile_bytes;
        const uint32_t sB_addr = smem_u32(sB);
        int s = 0, a = 0;
        uint32_t full_par = 0, acc_par = 1;
        for (int it = 0; it < my_tiles; ++it) {
            const int t = t0 + it;
            bool ok = true;
            if (t >= req_end) {
                // first block of another request: wait until the epilogue warps have rebuilt the A operand
                while (t >= req_end) {
                    ++req;
                    req_end = __ldg(p.offsets + req + 1);
                }
                ok = mbar_wait(&bars->a_ready, a_gen & 1u);
                ++a_gen;
            }
            if (ok) ok = mbar_wait(&bars->full[s], full_par);
            if (!ok || !mbar_wait(&bars->acc_empty[a], acc_par)) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 5);
                break;
            }
            tc_fence_after();
            const uint32_t b_addr = sB_addr + (uint32_t)(s * tile_bytes);
            const uint32_t d_base = tmem_base + (uint32_t)(a * acc_cols);
            if constexpr (NM > 0) {
                umma_f16_block16<NM>(d_base, a_lo, (uint32_t)smem_desc_sw128(b_addr), desc_hi, idesc);
            } else {
                for (int g = 0; g < p.G; ++g)
                    for (int kc = 0; kc < p.cpg; ++kc) {
                        const int c = g * p.cpg + kc;
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            umma_f16(d_base + (uint32_t)(g * p.M), smem_desc_sw128(a_addr + (uint32_t)(c * kChunkA + k4 * 32)),
                                     smem_desc_sw128(b_addr + (uint32_t)(c * chunk_b + k4 * 32)), idesc, (kc | k4) ? 1u : 0u);
                    }
            }
            // one commit per block: the epilogue set that receives it passes the "shared memory is free" half
            // of the news on to the producer
            umma_commit(&bars->acc_full[a]);
            if (++s == stages) {
                s = 0;
                full_par ^= 1u;
            }
            if (++a == n_acc) {
                a = 0;
                acc_par ^= 1u;
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue: block-local softmax pieces
        // Two sets of four warps take alternate blocks, so each scheduler holds two epilogue warps and
        // one can compute while the other waits for tensor memory.  With four accumulator sets the MMA
        // warp runs two blocks ahead of each epilogue set, which then never waits for the tensor core.
        const int set = (warp - 2) >> 2;
        const int qd = warp & 3;                 // the TMEM lane quarter this warp may read
        const int row = qd * 32 + lane;
        const int hl = row / p.Rp, j = row - hl * p.Rp;
        int req = 0, req_end = 0, nrows = 0;
        if (my_tiles > 0) {
            req = find_request(p.offsets, p.n_req, t0);
            req_end = __ldg(p.offsets + req + 1);
            nrows = (__ldg(p.q_offsets + req + 1) - __ldg(p.q_offsets + req)) * p.gq;
        }
        const int cpm = p.M >> 5;                // 32-column chunks per group
        const int n_loads = p.G * 2 * cpm;       // per group: one sweep for the maximum, one for the exponentials
        int sfree = set % p.stages;               // stage of this set's current block
        for (int it = set; it < my_tiles; it += 2) {
            const int a = it % p.n_acc;
            const int t = t0 + it;
            const int slot = p.slot_ids ? __ldg(p.slot_ids + t) : t;   // needed only at the end: in flight during the wait
            if (t >= req_end) {
                while (t >= req_end) {
                    ++req;
                    req_end = __ldg(p.offsets + req + 1);
                }
                nrows = (__ldg(p.q_offsets + req + 1) - __ldg(p.q_offsets + req)) * p.gq;
            }
            if (!mbar_wait(&bars->acc_full[a], (uint32_t)((it / p.n_acc) & 1))) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 5);
                break;
            }
            if (*(volatile int32_t*)&bars->abort_flag) break;
            tc_fence_after();
            if (qd == 0 && lane == 0) mbar_arrive(&bars->empty[sfree]);   // the MMAs have read the block's shared memory
            sfree += 2;
            while (sfree >= p.stages) sfree -= p.stages;
            // every MMA issued so far has completed.  If the next block belongs to another request, its
            // A operand is built now, before this block's exponentials, so the tensor core is not kept waiting
            if (it + 1 < my_tiles && t + 1 >= req_end) {
                int nreq = req, nend = req_end;
                while (t + 1 >= nend) {
                    ++nreq;
                    nend = __ldg(p.offsets + nreq + 1);
                }
                build_a_operand(sA, p, nreq, row);
                fence_proxy_async();
                mbar_arrive(&bars->a_ready);
            }
            const bool live = hl < p.hpg && j < nrows;
            const uint32_t tbase = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(a * acc_cols);
            float2* orow = p.part + (int64_t)t * p.Rtot + hl * p.Rp + j;
            // The loads of one block form a sequence (group, sweep, chunk); the next one is in flight
            // while the current one is consumed.
            float mx = -INFINITY, mb = 0.0f, s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
            // load i of the sequence: group i / (2*cpm), sweep (i / cpm) & 1, chunk i % cpm (counters, no divisions)
            int ag = 0, ar = 0;                  // position of the next load to issue
            auto next_address = [&]() {
                const int c = ar >= cpm ? ar - cpm : ar;
                const uint32_t adr = tbase + (uint32_t)(ag * p.M + c * 32);
                if (++ar == 2 * cpm) {
                    ar = 0;
                    ++ag;
                }
                return adr;
            };
            int cg = 0, cr = 0;                  // position of the next load to consume
            auto consume = [&](const uint32_t (&v)[32]) {
                if (cr < cpm) {
                    float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        m0 = fmaxf(m0, __uint_as_float(v[e]));
                        m1 = fmaxf(m1, __uint_as_float(v[e + 1]));
                        m2 = fmaxf(m2, __uint_as_float(v[e + 2]));
                        m3 = fmaxf(m3, __uint_as_float(v[e + 3]));
                    }
                    mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                    if (cr == cpm - 1) mb = mx * kLog2e;        // the block maximum, in units of log2
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        s0 += ex2(fmaf(__uint_as_float(v[e]), kLog2e, -mb));
                        s1 += ex2(fmaf(__uint_as_float(v[e + 1]), kLog2e, -mb));
                        s2 += ex2(fmaf(__uint_as_float(v[e + 2]), kLog2e, -mb));
                        s3 += ex2(fmaf(__uint_as_float(v[e + 3]), kLog2e, -mb));
                    }
                }
                if (++cr == 2 * cpm) {
                    if (live) {
                        float2 o = make_float2(mb, (s0 + s1) + (s2 + s3));
                        if (slot < 0) o = make_float2(-INFINITY, 0.0f);
                        orow[cg * p.hpg * p.Rp] = o;
                    }
                    mx = -INFINITY;
                    s0 = s1 = s2 = s3 = 0.0f;
                    cr = 0;
                    ++cg;
                }
            };
            if (p.M == 64) {
                // one block of one group fits in registers: a single read of tensor memory serves both the
                // maximum and the exponentials
                for (int g = 0; g < p.G; ++g) {
                    uint32_t v[64];
                    tmem_ld64(tbase + (uint32_t)(g * 64), v);
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 64; e += 4) {
                        m0 = fmaxf(m0, __uint_as_float(v[e]));
                        m1 = fmaxf(m1, __uint_as_float(v[e + 1]));
                        m2 = fmaxf(m2, __uint_as_float(v[e + 2]));
                        m3 = fmaxf(m3, __uint_as_float(v[e + 3]));
                    }
                    const float nb = -(fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * kLog2e);
                    float q0 = 0.0f, q1 = 0.0f, q2 = 0.0f, q3 = 0.0f;
#pragma unroll
                    for (int e = 0; e < 64; e += 4) {
                        q0 += ex2(fmaf(__uint_as_float(v[e]), kLog2e, nb));
                        q1 += ex2(fmaf(__uint_as_float(v[e + 1]), kLog2e, nb));
                        q2 += ex2(fmaf(__uint_as_float(v[e + 2]), kLog2e, nb));
                        q3 += ex2(fmaf(__uint_as_float(v[e + 3]), kLog2e, nb));
                    }
                    if (live) {
                        float2 o = make_float2(-nb, (q0 + q1) + (q2 + q3));
                        if (slot < 0) o = make_float2(-INFINITY, 0.0f);
                        orow[g * p.hpg * p.Rp] = o;
                    }
                }
                tc_fence_before();
                mbar_arrive(&bars->acc_empty[a]);
                continue;
            }
            uint32_t va[32], vb[32];
            tmem_ld32_issue(next_address(), va);
            for (int i = 0; i < n_loads; i += 2) {
                tmem_ld_wait(va);
                tmem_ld32_issue(next_address(), vb);
                consume(va);
                tmem_ld_wait(vb);
                if (i + 2 < n_loads) tmem_ld32_issue(next_address(), va);
                consume(vb);
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[a]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ------------------------------------------------------------------------------ pass 1, two blocks per instruction
// The same pipeline for the common shape (64 positions per block, heads * d_pruned == 256, two head
// groups), with consecutive candidate blocks of one request taken in pairs: an M128 N128 K16 instruction
// costs hardly more than an N64 one, so the sixteen instructions of a tile now cover two blocks, and the
// MMA-issuing thread - the serial resource of the one-block kernel - has half the work per block.  A pair
// never spans two requests (they have different A operands); a request's odd block is a tile of one.
// Two stages of 64 KiB, two accumulator sets of 2 x 128 columns.
constexpr int kPairStage = 65536;
__global__ void __launch_bounds__(kTcThreads, 1)
kvstar_partial_pair_kernel(const __grid_constant__ CUtensorMap tmap, KsParams p)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // pointer arithmetic keeps the shared address space
    unsigned char* sA = smem;                                  // 4 chunks of 16 KiB
    unsigned char* sB = sA + 4 * kChunkA;                      // 2 stages: chunk c at c*16 KiB, second block 8 KiB further
    KsBarriers* bars = reinterpret_cast<KsBarriers*>(sB + 2 * kPairStage);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = (int)((int64_t)p.total * blockIdx.x / gridDim.x);
    const int t1 = (int)((int64_t)p.total * (blockIdx.x + 1) / gridDim.x);
    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
            mbar_init(&bars->acc_full[s], 1);
            mbar_init(&bars->acc_empty[s], 128);
        }
        mbar_init(&bars->a_ready, 128);
        bars->abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (t1 > t0 && tid < kRows) build_a_operand(sA, p, find_request(p.offsets, p.n_req, t0), tid);
    fence_proxy_async();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    // every role walks the same tiling: (first block t, blocks in the tile nb, request, its end)
    int req = 0, req_end = 0;
    if (t1 > t0) {
        req = find_request(p.offsets, p.n_req, t0);
        req_end = __ldg(p.offsets + req + 1);
    }
    auto enter = [&](int t) {          // request of block t (t is never inside an empty request's range)
        bool changed = false;
        while (t >= req_end) {
            ++req;
            req_end = __ldg(p.offsets + req + 1);
            changed = true;
        }
        return changed;
    };
    auto blocks_of = [&](int t) { return (t + 1 < req_end && t + 1 < t1) ? 2 : 1; };

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------------ TMA producer
        int it = 0;
        for (int t = t0; t < t1; ++it) {
            enter(t);
            const int nb = blocks_of(t);
            const int s = it & 1;
            int slot[2];
            for (int h = 0; h < nb; ++h) slot[h] = p.slot_ids ? __ldg(p.slot_ids + t + h) : t + h;   // in flight during the wait
            if (!mbar_wait(&bars->empty[s], (uint32_t)(((it >> 1) & 1) ^ 1))) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 5);
                break;
            }
            if (*(volatile int32_t*)&bars->abort_flag) break;
            unsigned char* dst = sB + (size_t)s * kPairStage;
            mbar_expect_tx(&bars->full[s], (uint32_t)(nb * 32768));
            for (int h = 0; h < nb; ++h)
#pragma unroll
                for (int c = 0; c < 4; ++c) tma_load_2d(dst + c * 16384 + h * 8192, &tmap, c * 64, slot[h] * 64, &bars->full[s]);
            t += nb;
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const uint32_t a_lo = (uint32_t)smem_desc_sw128(smem_u32(sA));
        const uint32_t desc_hi = (uint32_t)(smem_desc_sw128(0) >> 32);
        const uint32_t idesc2 = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        const uint32_t idesc1 = (1u << 4) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        const uint32_t sB_addr = smem_u32(sB);
        uint32_t a_gen = 0;
        int it = 0;
        for (int t = t0; t < t1; ++it) {
            bool ok = true;
            if (enter(t)) {            // first block of another request: the epilogue warps have to rebuild the A operand first
                ok = mbar_wait(&bars->a_ready, a_gen & 1u);
                ++a_gen;
            }
            const int nb = blocks_of(t);
            const int s = it & 1;
            const uint32_t par = (uint32_t)((it >> 1) & 1);
            if (!ok || !mbar_wait(&bars->full[s], par) || !mbar_wait(&bars->acc_empty[s], par ^ 1u)) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 5);
                break;
            }
            tc_fence_after();
            umma_f16_block16<2, 128>(tmem_base + (uint32_t)(s * 256), a_lo, (uint32_t)smem_desc_sw128(sB_addr + (uint32_t)(s * kPairStage)),
                                     desc_hi, nb == 2 ? idesc2 : idesc1);
            umma_commit(&bars->acc_full[s]);
            t += nb;
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue (two sets, alternate tiles)
        const int set = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        const int hl = row / p.Rp, j = row - hl * p.Rp;
        int nrows = t1 > t0 ? (__ldg(p.q_offsets + req + 1) - __ldg(p.q_offsets + req)) * p.gq : 0;
        int it = 0;
        for (int t = t0; t < t1; ++it) {
            if (enter(t)) nrows = (__ldg(p.q_offsets + req + 1) - __ldg(p.q_offsets + req)) * p.gq;
            const int nb = blocks_of(t);
            if ((it & 1) != set) {
                t += nb;
                continue;
            }
            const int s = it & 1;                               // == set: stage and accumulator set of this tile
            int slot[2];
            for (int h = 0; h < nb; ++h) slot[h] = p.slot_ids ? __ldg(p.slot_ids + t + h) : t + h;
            if (!mbar_wait(&bars->acc_full[s], (uint32_t)((it >> 1) & 1))) {
                bars->abort_flag = 1;
                if (p.err) atomicExch(p.err, 5);
                break;
            }
            if (*(volatile int32_t*)&bars->abort_flag) break;
            tc_fence_after();
            if (qd == 0 && lane == 0) mbar_arrive(&bars->empty[s]);   // the MMAs have read the tile's shared memory
            // every MMA issued so far has completed: if the next tile starts another request, build its A operand now
            const int tn = t + nb;
            if (tn < t1 && tn >= req_end) {
                int nreq = req, nend = req_end;
                while (tn >= nend) {
                    ++nreq;
                    nend = __ldg(p.offsets + nreq + 1);
                }
                build_a_operand(sA, p, nreq, row);
                fence_proxy_async();
                mbar_arrive(&bars->a_ready);
            }
            const bool live = hl < p.hpg && j < nrows;
            const uint32_t tbase = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(s * 256);
            for (int h = 0; h < nb; ++h) {
                float2* orow = p.part + (int64_t)(t + h) * p.Rtot + hl * p.Rp + j;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    uint32_t v[64];
                    tmem_ld64(tbase + (uint32_t)(g * 128 + h * 64), v);
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 64; e += 4) {
                        m0 = fmaxf(m0, __uint_as_float(v[e]));
                        m1 = fmaxf(m1, __uint_as_float(v[e + 1]));
                        m2 = fmaxf(m2, __uint_as_float(v[e + 2]));
                        m3 = fmaxf(m3, __uint_as_float(v[e + 3]));
                    }
                    const float nbias = -(fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * kLog2e);
                    float q0 = 0.0f, q1 = 0.0f, q2 = 0.0f, q3 = 0.0f;
#pragma unroll
                    for (int e = 0; e < 64; e += 4) {
                        q0 += ex2(fmaf(__uint_as_float(v[e]), kLog2e, nbias));
                        q1 += ex2(fmaf(__uint_as_float(v[e + 1]), kLog2e, nbias));
                        q2 += ex2(fmaf(__uint_as_float(v[e + 2]), kLog2e, nbias));
                        q3 += ex2(fmaf(__uint_as_float(v[e + 3]), kLog2e, nbias));
                    }
                    if (live) {
                        float2 o = make_float2(-nbias, (q0 + q1) + (q2 + q3));
                        if (slot[h] < 0) o = make_float2(-INFINITY, 0.0f);
                        orow[g * p.hpg * p.Rp] = o;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[s]);
            t += nb;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ------------------------------------------------------------------------------ pass 1, CUDA cores
// Any shape: one CTA per candidate block, the block's representations in shared memory, one thread
// per query row at a time; dot products as fp32 fused multiply-adds in channel order.
__global__ void __launch_bounds__(256)
kvstar_partial_generic_kernel(KsParams p)
{
    extern __shared__ __align__(16) unsigned char smem_g[];
    uint16_t* sk = reinterpret_cast<uint16_t*>(smem_g);     // [M][H][dp]
    const int t = blockIdx.x;
    int slot = p.slot_ids ? __ldg(p.slot_ids + t) : t;
    if (slot >= 0 && slot >= p.n_slots) {                    // outside the table: reported, treated as an empty entry
        if (p.err && threadIdx.x == 0) atomicExch(p.err, 3);
        slot = -1;
    }
    const int req = find_request(p.offsets, p.n_req, t);
    const int q0 = __ldg(p.q_offsets + req), nx = min(__ldg(p.q_offsets + req + 1) - q0, p.Rp / p.gq);
    const int n_el = p.M * p.C;
    if (slot >= 0) {
        const uint4* src = reinterpret_cast<const uint4*>(p.reps + (int64_t)slot * n_el);
        for (int i = threadIdx.x; i < n_el / 8; i += blockDim.x) reinterpret_cast<uint4*>(sk)[i] = __ldg(src + i);
    }
    __syncthreads();
    for (int r = threadIdx.x; r < nx * p.Hq; r += blockDim.x) {
        const int xq = r / p.Hq, hq = r - xq * p.Hq;
        const int h = hq / p.gq, gg = hq - h * p.gq;
        float2 o = make_float2(-INFINITY, 0.0f);
        if (slot >= 0) {
            const uint16_t* qrow = p.q + ((int64_t)(q0 + xq) * p.Hq + hq) * p.d_orig;
            const int64_t* pr = p.pruned ? p.pruned + ((int64_t)req * p.H + h) * p.dp : nullptr;
            float mx = -INFINITY;
            for (int pass = 0; pass < 2; ++pass) {
                float sum = 0.0f;
                for (int m = 0; m < p.M; ++m) {
                    const uint16_t* kv = sk + ((size_t)m * p.H + h) * p.dp;
                    float acc = 0.0f;
                    for (int d = 0; d < p.dp; ++d) {
                        const uint16_t qb = __ldg(qrow + (pr ? __ldg(pr + d) : d));
                        acc = fmaf(__half2float(__ushort_as_half(qb)), __half2float(__ushort_as_half(kv[d])), acc);
                    }
                    if (pass == 0) mx = fmaxf(mx, acc);
                    else sum += ex2(fmaf(acc, kLog2e, -mx * kLog2e));
                }
                if (pass == 1) o = make_float2(mx * kLog2e, sum);
            }
        }
        p.part[(int64_t)t * p.Rtot + h * p.Rp + xq * p.gq + gg] = o;
    }
}

// ------------------------------------------------------------------------------ pass 2a: row statistics
// grid (row groups of 32, requests); lanes are rows, the 8 warps split the request's blocks and merge
// their running (max, sum) pairs through shared memory.
__global__ void __launch_bounds__(256)
kvstar_stats_kernel(KsParams p)
{
    __shared__ float2 sm[8][32];
    const int req = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rowid = blockIdx.x * 32 + lane;
    const int b0 = __ldg(p.offsets + req), b1 = __ldg(p.offsets + req + 1);
    const int nrows = (__ldg(p.q_offsets + req + 1) - __ldg(p.q_offsets + req)) * p.gq;
    const bool live = rowid < p.Rtot && (rowid % p.Rp) < nrows;
    float m = -INFINITY, z = 0.0f;
    if (live) {
        // eight independent loads per step, then one branch-free merge: the loop is bound by memory
        // latency, so the loads must not wait for the running pair
        for (int b = b0 + warp * 8; b < b1; b += 64) {
            float2 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = b + u < b1 ? __ldcg(p.part + (int64_t)(b + u) * p.Rtot + rowid) : make_float2(-INFINITY, 0.0f);
            float mn = m;
#pragma unroll
            for (int u = 0; u < 8; ++u) mn = fmaxf(mn, v[u].x);
            const float ms = mn == -INFINITY ? 0.0f : mn;      // keeps (-inf) - (-inf) out of the exponent
            float acc = z * ex2(m - ms);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += v[u].y * ex2(v[u].x - ms);
            z = acc;
            m = mn;
        }
    }
    sm[warp][lane] = make_float2(m, z);
    __syncthreads();
    if (warp == 0 && rowid < p.Rtot) {
        float mm = -INFINITY;
        for (int w = 0; w < 8; ++w) mm = fmaxf(mm, sm[w][lane].x);
        float zz = 0.0f;
        for (int w = 0; w < 8; ++w)
            if (sm[w][lane].x > -INFINITY) zz += sm[w][lane].y * ex2(sm[w][lane].x - mm);
        p.stats[(int64_t)req * p.Rtot + rowid] = make_float2(mm, zz > 0.0f ? 1.0f / zz : 0.0f);
    }
}

// ------------------------------------------------------------------------------ pass 2b: votes
// one warp per candidate block
__global__ void __launch_bounds__(256)
kvstar_vote_kernel(KsParams p)
{
    __shared__ int s_off[1025], s_q[1025];
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    const bool cached = p.n_req <= 1024;       // request boundaries and query counts, searched in shared memory
    if (cached)
        for (int i = threadIdx.x; i <= p.n_req; i += blockDim.x) {
            s_off[i] = __ldg(p.offsets + i);
            s_q[i] = __ldg(p.q_offsets + i);
        }
    __syncthreads();
    if (t >= p.total) return;
    int req, nrows;
    if (cached) {
        int lo = 0, hi = p.n_req;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= t) lo = mid; else hi = mid;
        }
        req = lo;
        nrows = (s_q[req + 1] - s_q[req]) * p.gq;
    } else {
        req = find_request(p.offsets, p.n_req, t);
        nrows = (__ldg(p.q_offsets + req + 1) - __ldg(p.q_offsets + req)) * p.gq;
    }
    const float2* pp = p.part + (int64_t)t * p.Rtot;
    const float2* st = p.stats + (int64_t)req * p.Rtot;
    float acc = 0.0f;
    for (int r0 = lane; r0 < p.Rtot; r0 += 256) {
        // eight independent pairs of loads before the first use
        float2 v[8], sr[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int r = r0 + u * 32;
            const bool on = r < p.Rtot && (r % p.Rp) < nrows;
            v[u] = on ? __ldcg(pp + r) : make_float2(-INFINITY, 0.0f);
            sr[u] = on ? __ldcg(st + r) : make_float2(0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (v[u].x > -INFINITY) acc += v[u].y * ex2(v[u].x - sr[u].x) * sr[u].y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) p.out[t] = acc;
}

// ------------------------------------------------------------------------------ block representations
// CTA per block; 16 tokens at a time are staged with coalesced 16-byte loads, then each thread
// produces kept channels: fp32 sum of `merge` tokens in order, times 1/merge, rounded to bf16 (the
// cache's dtype, as torch's mean does), then converted to half.
struct ReprParams {
    const uint16_t* k;
    ucmx_kv_geometry g;
    const int32_t* ids;
    const int32_t* out_slots;
    int64_t out_rows;
    int32_t* err;
    const int64_t* pruned;
    uint16_t* out;
    int32_t dp, merge, M;
};

__global__ void __launch_bounds__(256)
kvstar_block_repre_kernel(ReprParams p)
{
    extern __shared__ __align__(16) unsigned char smem_r[];
    uint16_t* st = reinterpret_cast<uint16_t*>(smem_r);     // [tokens_per_step][H*D]
    const int i = blockIdx.x;
    const int id = checked_block_id(p.ids, i, p.g.reserved, p.err);
    const int64_t slot = id < 0 ? -1 : checked_out_row(p.out_slots, i, p.out_rows, p.err);
    if (id < 0 || slot < 0) return;
    const int E = p.g.n_kv_heads * p.g.head_dim;
    const int C = p.g.n_kv_heads * p.dp;
    const int step_m = max(1, 16 / p.merge);                // output rows per step
    const float inv = 1.0f / (float)p.merge;
    const uint16_t* blk = p.k + (int64_t)id * p.g.block_stride;
    for (int m0 = 0; m0 < p.M; m0 += step_m) {
        const int rows = min(step_m, p.M - m0) * p.merge;
        for (int u = threadIdx.x; u < rows * (E / 8); u += blockDim.x) {
            const int tr = u / (E / 8), c = u - tr * (E / 8);
            reinterpret_cast<uint4*>(st)[u] =
                __ldg(reinterpret_cast<const uint4*>(blk + (int64_t)(m0 * p.merge + tr) * p.g.token_stride) + c);
        }
        __syncthreads();
        for (int o = threadIdx.x; o < (rows / p.merge) * C; o += blockDim.x) {
            const int mr = o / C, hc = o - mr * C;
            const int h = hc / p.dp, dpi = hc - h * p.dp;
            const int d = p.pruned ? (int)__ldg(p.pruned + (int64_t)h * p.dp + dpi) : dpi;
            float acc = 0.0f;
            for (int c = 0; c < p.merge; ++c) acc += bf16lo((uint32_t)st[(size_t)(mr * p.merge + c) * E + h * p.g.head_dim + d]);
            const float rounded = __bfloat162float(__float2bfloat16_rn(acc * inv));
            p.out[((int64_t)slot * p.M + (m0 + mr)) * C + hc] = __half_as_ushort(__float2half_rn(rounded));
        }
        __syncthreads();
    }
}

int row_pad(int rows)
{
    if (rows > kRows) return rows;
    int r = 1;
    while (r < rows) r <<= 1;
    return r;
}

}  // namespace
}  // namespace ucmx

using namespace ucmx;

extern "C" int32_t ucmx_kvstar_block_repre(const void* k_cache, const ucmx_kv_geometry* geom, const int32_t* block_ids,
                                           const int32_t* out_slots, int64_t n_out_slots, int32_t n,
                                           const int64_t* pruned_index, int32_t d_pruned, int32_t merge, void* reps_f16,
                                           ucmx_stream_t stream)
{
    if (n < 0) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (!geom || geom->reserved < 1 || n_out_slots < 1) return UCMX_EPARAM;
    if (!k_cache || !geom || !block_ids || !reps_f16 || merge < 1 || d_pruned < 1) return UCMX_EPARAM;
    const int T = geom->block_tokens, H = geom->n_kv_heads, D = geom->head_dim;
    if (T < 1 || H < 1 || D < 8 || (D & 7) || T % merge || d_pruned > D || (!pruned_index && d_pruned != D)) return UCMX_EPARAM;
    if ((geom->token_stride & 7) || (geom->block_stride & 7) || ((uintptr_t)k_cache & 15)) return UCMX_EPARAM;
    ReprParams p{};
    p.k = (const uint16_t*)k_cache;
    p.g = *geom;
    p.ids = block_ids;
    p.out_slots = out_slots;
    p.out_rows = n_out_slots;
    p.err = error_word();
    p.pruned = pruned_index;
    p.out = (uint16_t*)reps_f16;
    p.dp = d_pruned;
    p.merge = merge;
    p.M = T / merge;
    const int step_t = (16 / merge > 0 ? 16 / merge : 1) * merge;
    const size_t smem = (size_t)step_t * H * D * 2;
    if (smem > 200 * 1024) return UCMX_EUNSUPPORTED;
    UCMX_CUDA(cudaFuncSetAttribute(kvstar_block_repre_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kvstar_block_repre_kernel<<<n, 256, smem, (cudaStream_t)stream>>>(p);
    UCMX_LAUNCH_CHECK("kvstar_block_repre_kernel");
    return UCMX_OK;
}

namespace ucmx {
namespace {
// Does the shape take the tensor-core kernels, and which one: 0 = no (CUDA-core kernel), 1 = one block per tile,
// 2 = two blocks per instruction.  Needs p.M, p.H, p.dp, p.C, p.Rp; fills the tiling fields of p.
int plan_tensor_core(KsParams& p, int64_t n_slots)
{
    const int M = p.M, H = p.H, d_pruned = p.dp, C = p.C;
    // several heads per 128-row instruction, whole 64-element K chunks per head group
    bool tc = encode_fn() != nullptr && p.Rp <= kRows && (d_pruned % 16) == 0 && (M % 32) == 0 && M <= 256 &&
              (C % 64) == 0 && n_slots * M < 0x7fffffffll;
    if (!tc) return 0;
    p.hpg = kRows / p.Rp < H ? kRows / p.Rp : H;
    while (p.hpg > 1 && (H % p.hpg || (p.hpg * d_pruned) % 64)) --p.hpg;
    if (!(H % p.hpg == 0 && (p.hpg * d_pruned) % 64 == 0)) return 0;
    p.G = H / p.hpg;
    p.cpg = p.hpg * d_pruned / 64;
    if (p.G * M > 256) return 0;                 // two accumulator sets must fit the 512 TMEM columns
    p.n_acc = p.G * M <= 128 ? 4 : 2;
    p.tile_bytes = M * C * 2;
    const size_t a_bytes = (size_t)p.G * p.cpg * kChunkA;
    const int64_t budget = 220 * 1024 - 1024 - (int64_t)a_bytes - (int64_t)sizeof(KsBarriers) - 64;
    p.stages = budget > 0 ? (int)(budget / p.tile_bytes) : 0;
    if (p.stages > 8) p.stages = 8;
    if (p.stages < 2) return 0;                  // wide heads (no channel pruning) do not fit: CUDA-core kernel
    return (M == 64 && C == 256 && p.cpg == 2 && p.G == 2) ? 2 : 1;
}
}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_kvstar_kernel_choice(int32_t n_slots, int32_t M, int32_t n_kv_heads, int32_t d_pruned,
                                             int32_t max_q_tokens, int32_t n_q_heads)
{
    using namespace ucmx;
    if (M < 1 || n_kv_heads < 1 || d_pruned < 1 || n_q_heads < n_kv_heads || n_q_heads % n_kv_heads || max_q_tokens < 1)
        return UCMX_EPARAM;
    KsParams p{};
    p.M = M;
    p.H = n_kv_heads;
    p.dp = d_pruned;
    p.C = n_kv_heads * d_pruned;
    p.Rp = row_pad(max_q_tokens * (n_q_heads / n_kv_heads));
    return plan_tensor_core(p, n_slots);
}

extern "C" size_t ucmx_kvstar_workspace_bytes(int32_t total_blocks, int32_t n_req, int32_t max_q_tokens, int32_t n_q_heads,
                                              int32_t n_kv_heads)
{
    if (total_blocks < 0 || n_req < 0 || max_q_tokens < 1 || n_kv_heads < 1 || n_q_heads < n_kv_heads) return 0;
    const size_t rtot = (size_t)n_kv_heads * row_pad(max_q_tokens * (n_q_heads / n_kv_heads));
    return ((size_t)total_blocks + (size_t)n_req) * rtot * sizeof(float2) + 256;
}

extern "C" int32_t ucmx_kvstar_scores(const void* reps_f16, int32_t n_slots, int32_t M, int32_t n_kv_heads, int32_t d_pruned,
                                      const int32_t* req_offsets, const int32_t* slot_ids, int32_t n_req, int32_t total,
                                      const void* q_f16, const int32_t* q_offsets, int32_t max_q_tokens, int32_t n_q_heads,
                                      int32_t d_orig, const int64_t* pruned_index, void* workspace, size_t workspace_bytes,
                                      float* out_scores, ucmx_stream_t stream)
{
    if (n_req < 0 || total < 0) return UCMX_EPARAM;
    if (n_req == 0 || total == 0) return UCMX_OK;
    if (!reps_f16 || !req_offsets || !q_f16 || !q_offsets || !workspace || !out_scores) return UCMX_EPARAM;
    const int H = n_kv_heads;
    if (M < 1 || H < 1 || d_pruned < 1 || n_q_heads < H || n_q_heads % H || max_q_tokens < 1 || n_slots < 1) return UCMX_EPARAM;
    if (d_pruned > d_orig || (!pruned_index && d_pruned != d_orig)) return UCMX_EPARAM;
    const int C = H * d_pruned;
    if ((C & 7) || ((uintptr_t)reps_f16 & 15) || ((uintptr_t)q_f16 & 15) || (d_orig & 7)) return UCMX_EPARAM;
    if (workspace_bytes < ucmx_kvstar_workspace_bytes(total, n_req, max_q_tokens, n_q_heads, H)) return UCMX_EPARAM;
    cudaStream_t st = (cudaStream_t)stream;
    KsParams p{};
    p.q = (const uint16_t*)q_f16;
    p.q_offsets = q_offsets;
    p.pruned = pruned_index;
    p.reps = (const uint16_t*)reps_f16;
    p.offsets = req_offsets;
    p.slot_ids = slot_ids;
    p.n_slots = n_slots;
    p.n_req = n_req;
    p.total = total;
    p.M = M;
    p.H = H;
    p.dp = d_pruned;
    p.C = C;
    p.Hq = n_q_heads;
    p.gq = n_q_heads / H;
    p.d_orig = d_orig;
    p.Rp = row_pad(max_q_tokens * p.gq);
    p.Rtot = H * p.Rp;
    p.part = reinterpret_cast<float2*>(((uintptr_t)workspace + 255) & ~(uintptr_t)255);
    p.stats = p.part + (size_t)total * p.Rtot;
    p.out = out_scores;
    p.err = error_word();

    bool tc = plan_tensor_core(p, n_slots) != 0;
    if (tc) {
        p.idesc = (1u << 4) | ((uint32_t)(M >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);   // D fp32, A and B half, K-major
        const size_t a_bytes = (size_t)p.G * p.cpg * kChunkA;
        {
            alignas(64) CUtensorMap tmap;
            const cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)n_slots * M};
            const cuuint64_t strides[1] = {(cuuint64_t)C * 2};
            const cuuint32_t box[2] = {64, (cuuint32_t)M};
            const cuuint32_t es[2] = {1, 1};
            const CUresult r = encode_fn()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(reps_f16), dims, strides,
                                           box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r == CUDA_SUCCESS) {
                const size_t smem = 1024 + a_bytes + (size_t)p.stages * p.tile_bytes + sizeof(KsBarriers) + 64;
                int grid = sm_count();
                if (grid > total) grid = total;
                if (M == 64 && C == 256 && p.cpg == 2 && p.G == 2) {
                    const size_t psmem = 1024 + 4 * (size_t)kChunkA + 2 * (size_t)kPairStage + sizeof(KsBarriers) + 64;
                    UCMX_CUDA(cudaFuncSetAttribute(kvstar_partial_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)psmem));
                    int pgrid = sm_count();
                    if (pgrid > total) pgrid = total;
                    kvstar_partial_pair_kernel<<<pgrid, kTcThreads, psmem, st>>>(tmap, p);
                    UCMX_LAUNCH_CHECK("kvstar_partial_pair_kernel");
                    goto pass2;
                }
                const bool special = M == 64 && C == 256 && (p.cpg == 1 || p.cpg == 2);
                auto kern = !special ? kvstar_partial_tc_kernel<0> : p.cpg == 1 ? kvstar_partial_tc_kernel<1> : kvstar_partial_tc_kernel<2>;
                UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                kern<<<grid, kTcThreads, smem, st>>>(tmap, p);
                UCMX_LAUNCH_CHECK("kvstar_partial_tc_kernel");
            } else {
                tc = false;
            }
        }
    }
    if (!tc) {
        const size_t smem = (size_t)M * C * 2;
        if (smem > 200 * 1024) {
            set_last_text("kvstar: a block's representations do not fit in shared memory");
            return UCMX_EUNSUPPORTED;
        }
        UCMX_CUDA(cudaFuncSetAttribute(kvstar_partial_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kvstar_partial_generic_kernel<<<total, 256, smem, st>>>(p);
        UCMX_LAUNCH_CHECK("kvstar_partial_generic_kernel");
    }
pass2:
    kvstar_stats_kernel<<<dim3((p.Rtot + 31) / 32, n_req), 256, 0, st>>>(p);
    UCMX_LAUNCH_CHECK("kvstar_stats_kernel");
    kvstar_vote_kernel<<<(total + 7) / 8, 256, 0, st>>>(p);
    UCMX_LAUNCH_CHECK("kvstar_vote_kernel");
    return UCMX_OK;
}

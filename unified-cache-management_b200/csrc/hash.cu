// KVComp path: sign-bit hash codes (stage 1b) and Hamming-similarity block scores (stage 2b).
//
// hash_encode reproduces, bit for bit, the sign of an fp32 fused-multiply-add chain over the input
// dimension (the order the CPU checker fixes for HashEncoder.compute_hash,
// ucm/sparse/kvcomp/hash_encoder.py:119-149), so it runs on CUDA cores with a register-tiled
// 8-vector x 4-bit micro-kernel fed from shared memory.  Encoding happens when a block is dumped
// (prefill), not on the decode critical path.
//
// score_hamming streams each candidate block's packed token codes once (16 KiB per block) and
// reduces them with XOR + popcount; integer arithmetic, exact.  The reference's einsum pairs every
// query head with every key head; that sum is folded into four bit-sliced count planes of the
// query so that a key word costs five popcounts instead of one per query head.
#include <cstdlib>

#include "common.cuh"

namespace ucmx {
namespace {

// ------------------------------------------------------------------ hash encode

constexpr int kHashThreads = 256;
constexpr int kHashTile = 64;  // vectors per CTA iteration: 8 warps x 8 vectors

struct HashParams {
    const uint16_t* x;   // dense source (or paged cache base)
    int64_t x_stride;    // dense: elements between vectors
    int64_t n_vec;
    const uint16_t* w;   // [dim, bits]
    int32_t dim, bits;
    uint8_t* out;
    // paged source
    int32_t paged;
    const int32_t* ids;
    const int32_t* out_slots;
    int64_t cache_blocks, out_rows;   // paged: blocks in the cache, rows of the code table
    int32_t* err;
    int64_t block_stride, token_stride;
    int32_t T, H, head_major;
};

__device__ __forceinline__ void hash_locate(const HashParams& p, int64_t v, const uint16_t*& src, int64_t& orow)
{
    if (!p.paged) {
        src = p.x + v * p.x_stride;
        orow = v;
        return;
    }
    const int64_t per_block = (int64_t)p.T * p.H;
    const int64_t i = v / per_block;
    const int32_t rem = (int32_t)(v - i * per_block);
    const int32_t t = rem / p.H, h = rem - t * p.H;
    const int32_t id = checked_block_id(p.ids, i, p.cache_blocks, p.err);
    const int64_t slot = id < 0 ? -1 : checked_out_row(p.out_slots, i, p.out_rows, p.err);
    src = (id < 0) ? nullptr : p.x + (int64_t)id * p.block_stride + (int64_t)t * p.token_stride + (int64_t)h * p.dim;
    orow = (slot < 0) ? -1 : (p.head_major ? (slot * p.H + h) * p.T + t : slot * per_block + rem);
}

__global__ void __launch_bounds__(kHashThreads) hash_encode_kernel(HashParams p)
{
    extern __shared__ __align__(16) float hsm[];
    float* Ws = hsm;                              // [dim][bits]
    float* xs = hsm + (size_t)p.dim * p.bits;     // [dim][kHashTile]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int i = tid; i < p.dim * p.bits; i += kHashThreads) Ws[i] = __uint_as_float((uint32_t)__ldg(p.w + i) << 16);

    const int pieces_per_vec = p.dim / 8;
    const int64_t n_tiles = (p.n_vec + kHashTile - 1) / kHashTile;
    const int nbytes = p.bits / 8;

    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t v0 = tile * kHashTile;
        __syncthreads();  // previous tile fully consumed (and Ws written, first time round)
        for (int pid = tid; pid < kHashTile * pieces_per_vec; pid += kHashThreads) {
            const int vec = pid % kHashTile, piece = pid / kHashTile;
            const int64_t v = v0 + vec;
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (v < p.n_vec) {
                const uint16_t* src;
                int64_t orow;
                hash_locate(p, v, src, orow);
                if (src) raw = __ldg(reinterpret_cast<const uint4*>(src) + piece);
            }
            float* col = xs + (size_t)(piece * 8) * kHashTile + vec;
            col[0 * kHashTile] = bf16lo(raw.x);
            col[1 * kHashTile] = bf16hi(raw.x);
            col[2 * kHashTile] = bf16lo(raw.y);
            col[3 * kHashTile] = bf16hi(raw.y);
            col[4 * kHashTile] = bf16lo(raw.z);
            col[5 * kHashTile] = bf16hi(raw.z);
            col[6 * kHashTile] = bf16lo(raw.w);
            col[7 * kHashTile] = bf16hi(raw.w);
        }
        __syncthreads();

        for (int bg = 0; bg < p.bits / 128; ++bg) {
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
            const float* wcol = Ws + bg * 128 + 4 * lane;
            const float* xrow = xs + 8 * warp;
#pragma unroll 4
            for (int d = 0; d < p.dim; ++d) {
                const float4 wv = *reinterpret_cast<const float4*>(wcol + (size_t)d * p.bits);
                const float4 xa = *reinterpret_cast<const float4*>(xrow + (size_t)d * kHashTile);
                const float4 xb = *reinterpret_cast<const float4*>(xrow + (size_t)d * kHashTile + 4);
                const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    acc[i][0] = fmaf(xv[i], wv.x, acc[i][0]);
                    acc[i][1] = fmaf(xv[i], wv.y, acc[i][1]);
                    acc[i][2] = fmaf(xv[i], wv.z, acc[i][2]);
                    acc[i][3] = fmaf(xv[i], wv.w, acc[i][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                uint32_t nib = (acc[i][0] > 0.0f ? 1u : 0u) | (acc[i][1] > 0.0f ? 2u : 0u) |
                               (acc[i][2] > 0.0f ? 4u : 0u) | (acc[i][3] > 0.0f ? 8u : 0u);
                uint32_t word = nib << (4 * (lane & 7));
                word |= __shfl_xor_sync(0xffffffffu, word, 1);
                word |= __shfl_xor_sync(0xffffffffu, word, 2);
                word |= __shfl_xor_sync(0xffffffffu, word, 4);
                const int64_t v = v0 + 8 * warp + i;
                if ((lane & 7) == 0 && v < p.n_vec) {
                    const uint16_t* src;
                    int64_t orow;
                    hash_locate(p, v, src, orow);
                    if (orow >= 0 && src)
                        *reinterpret_cast<uint32_t*>(p.out + orow * nbytes + (size_t)(bg * 4 + (lane >> 3)) * 4) = word;
                }
            }
        }
    }
}

int32_t launch_hash(HashParams& p, cudaStream_t st)
{
    if (p.dim < 8 || p.dim % 8 || p.bits < 128 || p.bits % 128) return UCMX_EUNSUPPORTED;
    const size_t smem = ((size_t)p.dim * p.bits + (size_t)p.dim * kHashTile) * sizeof(float);
    if (smem > 200 * 1024) return UCMX_EUNSUPPORTED;
    UCMX_CUDA(cudaFuncSetAttribute(hash_encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t n_tiles = (p.n_vec + kHashTile - 1) / kHashTile;
    const int per_sm = smem <= 100 * 1024 ? 2 : 1;
    int64_t grid = (int64_t)sm_count() * per_sm;
    if (grid > n_tiles) grid = n_tiles;
    hash_encode_kernel<<<(unsigned)grid, kHashThreads, smem, st>>>(p);
    UCMX_LAUNCH_CHECK("hash_encode_kernel");
    return UCMX_OK;
}

// ------------------------------------------------------------------ Hamming scores

struct HamParams {
    const uint8_t* codes;
    int64_t n_slots;     // rows of the code table
    int32_t* err;
    const int32_t* offsets;
    const int32_t* slot_ids;
    const uint8_t* q_codes;
    int32_t* out;
    int32_t n_req, total, H, T, words;  // words = bits/32 per code
    int32_t nq, cross;
};

constexpr int kHamThreads = 256;

// carry-save adder on 32 bit columns at once: (h, l) = a + b + c
__device__ __forceinline__ void csa(uint32_t& h, uint32_t& l, uint32_t a, uint32_t b, uint32_t c)
{
    const uint32_t u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}

// bits == 128 (one uint4 per code).  One warp per candidate block.
template <bool CROSS>
__global__ void __launch_bounds__(kHamThreads, CROSS ? 2 : 4) score_hamming_kernel(HamParams p)
{
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int pieces = p.H * p.T;  // uint4 codes per block row
    const size_t row_bytes = (size_t)pieces * 16;
    const int bits = 128;

    for (int64_t c = w0; c < p.total; c += W) {
        const int r = find_request(p.offsets, p.n_req, (int)c);
        int slot = p.slot_ids ? __ldg(p.slot_ids + c) : (int)c;
        if (slot >= 0 && (int64_t)slot >= p.n_slots) {      // outside the table: reported, treated as empty
            if (p.err && lane == 0) atomicExch(p.err, 3);
            slot = -1;
        }
        if (slot < 0) {
            if (lane == 0) p.out[c] = INT32_MIN;
            continue;
        }
        const uint4* row = reinterpret_cast<const uint4*>(p.codes + (size_t)slot * row_bytes);
        const uint4* qc = reinterpret_cast<const uint4*>(p.q_codes + (size_t)r * p.nq * 16);
        long long ham_total = 0;  // sum over pairs of popcount(q xor k)
        long long pairs = 0;
        if (CROSS) {
            // bit-sliced count of set query bits per position: c_b = P0 + 2 P1 + 4 P2 + 8 P3
            uint32_t P[4][4];
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) P[a][b] = 0;
            int C = 0;
            for (int i = 0; i < p.nq; ++i) {
                const uint4 q = __ldg(qc + i);
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    uint32_t x = qw[wd];
                    C += __popc(x);
                    uint32_t carry = P[0][wd] & x;
                    P[0][wd] ^= x;
                    x = carry;
                    carry = P[1][wd] & x;
                    P[1][wd] ^= x;
                    x = carry;
                    carry = P[2][wd] & x;
                    P[2][wd] ^= x;
                    P[3][wd] ^= carry;
                }
            }
            int a0 = 0, a1 = 0, a2 = 0, a3 = 0, a4 = 0;
            if ((pieces & 255) == 0) {
                // Carry-save counting (Harley-Seal): the lane's key words of one word position are added
                // bit-column-wise into binary counter planes with LOP3 full adders, eight words at a
                // time, and popcounts are taken once per 32 words on the planes instead of five
                // times per word; this keeps the all-pairs form bound by HBM rather than by the
                // popcount pipe.  A lane sees pieces/32 words per position (a multiple of 8).
                for (int base_pc = 0; base_pc < pieces; base_pc += 32 * 32) {
                    uint32_t ones[4] = {0, 0, 0, 0}, twos[4] = {0, 0, 0, 0}, fours[4] = {0, 0, 0, 0};
                    uint32_t eights[4] = {0, 0, 0, 0}, sixteens[4] = {0, 0, 0, 0}, thirtytwos[4] = {0, 0, 0, 0};
                    const int groups = min(4, (pieces - base_pc) / 256);
                    for (int grp = 0; grp < groups; ++grp) {
                        uint4 k[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) k[j] = ld_stream16(row + base_pc + (grp * 8 + j) * 32 + lane);
#pragma unroll
                        for (int wd = 0; wd < 4; ++wd) {
                            uint32_t x[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) x[j] = wd == 0 ? k[j].x : wd == 1 ? k[j].y : wd == 2 ? k[j].z : k[j].w;
                            uint32_t twosA, twosB, foursA, foursB, e8;
                            csa(twosA, ones[wd], ones[wd], x[0], x[1]);
                            csa(twosB, ones[wd], ones[wd], x[2], x[3]);
                            csa(foursA, twos[wd], twos[wd], twosA, twosB);
                            csa(twosA, ones[wd], ones[wd], x[4], x[5]);
                            csa(twosB, ones[wd], ones[wd], x[6], x[7]);
                            csa(foursB, twos[wd], twos[wd], twosA, twosB);
                            csa(e8, fours[wd], fours[wd], foursA, foursB);
                            const uint32_t c16 = eights[wd] & e8;
                            eights[wd] ^= e8;
                            const uint32_t c32 = sixteens[wd] & c16;
                            sixteens[wd] ^= c16;
                            thirtytwos[wd] ^= c32;
                        }
                    }
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        const uint32_t plane[6] = {ones[wd], twos[wd], fours[wd], eights[wd], sixteens[wd], thirtytwos[wd]};
#pragma unroll
                        for (int l = 0; l < 6; ++l) {
                            a0 += __popc(plane[l]) << l;
                            a1 += __popc(plane[l] & P[0][wd]) << l;
                            a2 += __popc(plane[l] & P[1][wd]) << l;
                            a3 += __popc(plane[l] & P[2][wd]) << l;
                            a4 += __popc(plane[l] & P[3][wd]) << l;
                        }
                    }
                }
            } else {
#pragma unroll 4
            for (int pc = lane; pc < pieces; pc += 32) {
                const uint4 k = ld_stream16(row + pc);
                const uint32_t kw[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    a0 += __popc(kw[wd]);
                    a1 += __popc(kw[wd] & P[0][wd]);
                    a2 += __popc(kw[wd] & P[1][wd]);
                    a3 += __popc(kw[wd] & P[2][wd]);
                    a4 += __popc(kw[wd] & P[3][wd]);
                }
            }
            }
            // sum_i popcount(q_i xor k) = C + nq*popc(k) - 2*sum_p 2^p popc(k & P_p)
            const long long weighted = (long long)a1 + 2ll * a2 + 4ll * a3 + 8ll * a4;
            long long lane_sum = (long long)p.nq * a0 - 2ll * weighted;
            int lo = (int)lane_sum;  // |lane_sum| < 2^31 for any realistic block
            lo = warp_sum_i(lo);
            ham_total = (long long)lo + (long long)pieces * C;
            pairs = (long long)pieces * p.nq;
        } else {
            int acc = 0;
            if ((p.T & 31) == 0) {
                for (int j = 0; j < p.H; ++j) {
                    const uint4 q = __ldg(qc + j);
                    const uint4* hrow = row + (size_t)j * p.T;
#pragma unroll 4
                    for (int s = lane; s < p.T; s += 32) {
                        const uint4 k = ld_stream16(hrow + s);
                        acc += __popc(k.x ^ q.x) + __popc(k.y ^ q.y) + __popc(k.z ^ q.z) + __popc(k.w ^ q.w);
                    }
                }
            } else {
                for (int pc = lane; pc < pieces; pc += 32) {
                    const uint4 q = __ldg(qc + pc / p.T);
                    const uint4 k = ld_stream16(row + pc);
                    acc += __popc(k.x ^ q.x) + __popc(k.y ^ q.y) + __popc(k.z ^ q.z) + __popc(k.w ^ q.w);
                }
            }
            ham_total = warp_sum_i(acc);
            pairs = pieces;
        }
        if (lane == 0) p.out[c] = (int32_t)(pairs * bits - 2 * ham_total);
    }
}

// any bits (multiple of 32): straightforward loop over query heads; used when bits != 128
__global__ void __launch_bounds__(kHamThreads) score_hamming_generic_kernel(HamParams p)
{
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t W = (int64_t)gridDim.x * warps_per_cta;
    const int64_t w0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int codes_per_row = p.H * p.T;
    const int64_t words_per_row = (int64_t)codes_per_row * p.words;
    for (int64_t c = w0; c < p.total; c += W) {
        const int r = find_request(p.offsets, p.n_req, (int)c);
        int slot = p.slot_ids ? __ldg(p.slot_ids + c) : (int)c;
        if (slot >= 0 && (int64_t)slot >= p.n_slots) {      // outside the table: reported, treated as empty
            if (p.err && lane == 0) atomicExch(p.err, 3);
            slot = -1;
        }
        if (slot < 0) {
            if (lane == 0) p.out[c] = INT32_MIN;
            continue;
        }
        const uint32_t* row = reinterpret_cast<const uint32_t*>(p.codes) + (size_t)slot * words_per_row;
        const uint32_t* qc = reinterpret_cast<const uint32_t*>(p.q_codes) + (size_t)r * p.nq * p.words;
        int acc = 0;
        for (int64_t wi = lane; wi < words_per_row; wi += 32) {
            const uint32_t k = __ldg(row + wi);
            const int code = (int)(wi / p.words), wd = (int)(wi - (int64_t)code * p.words);
            if (p.cross) {
                for (int i = 0; i < p.nq; ++i) acc += __popc(k ^ __ldg(qc + i * p.words + wd));
            } else {
                acc += __popc(k ^ __ldg(qc + (code / p.T) * p.words + wd));
            }
        }
        const long long ham = warp_sum_i(acc);
        const long long pairs = (long long)codes_per_row * (p.cross ? p.nq : 1);
        if (lane == 0) p.out[c] = (int32_t)(pairs * p.words * 32 - 2 * ham);
    }
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_hash_encode(const void* x, int64_t n_vec, int64_t x_stride, const void* w, int32_t dim,
                                    int32_t bits, uint8_t* out, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_vec < 0) return UCMX_EPARAM;
    if (n_vec == 0) return UCMX_OK;
    if (!x || !w || !out || x_stride < dim || (x_stride % 8) || ((uintptr_t)x & 15) || ((uintptr_t)out & 3))
        return UCMX_EPARAM;
    {
        const int32_t rc = hash_encode_tc(x, n_vec, x_stride, nullptr, nullptr, nullptr, 0, 0, w, dim, bits, 0, out,
                                          (cudaStream_t)stream);
        if (rc != UCMX_EUNSUPPORTED) return rc;
    }
    HashParams p{};
    p.x = (const uint16_t*)x;
    p.x_stride = x_stride;
    p.n_vec = n_vec;
    p.w = (const uint16_t*)w;
    p.dim = dim;
    p.bits = bits;
    p.out = out;
    p.paged = 0;
    return launch_hash(p, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_hash_encode_blocks(const void* k_cache, const ucmx_kv_geometry* g, const int32_t* block_ids,
                                           const int32_t* out_slots, int64_t n_out_slots, int32_t n, const void* w,
                                           int32_t bits, int32_t head_major, uint8_t* out, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n < 0 || !g) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (g->reserved < 1 || n_out_slots < 1) {
        set_last_text("hash_encode_blocks: the geometry must carry the number of blocks in the cache and the call the rows of the table");
        return UCMX_EPARAM;
    }
    if (!k_cache || !block_ids || !w || !out || ((uintptr_t)k_cache & 15) || ((uintptr_t)out & 3)) return UCMX_EPARAM;
    if (g->block_tokens < 1 || g->n_kv_heads < 1 || g->head_dim < 8) return UCMX_EPARAM;
    if ((g->token_stride % 8) || (g->block_stride % 8) || (g->head_dim % 8)) return UCMX_EPARAM;
    {
        const int32_t rc = hash_encode_tc(k_cache, 0, 0, g, block_ids, out_slots, n_out_slots, n, w, g->head_dim, bits,
                                          head_major, out, (cudaStream_t)stream);
        if (rc != UCMX_EUNSUPPORTED) return rc;
    }
    HashParams p{};
    p.x = (const uint16_t*)k_cache;
    p.n_vec = (int64_t)n * g->block_tokens * g->n_kv_heads;
    p.w = (const uint16_t*)w;
    p.dim = g->head_dim;
    p.bits = bits;
    p.out = out;
    p.paged = 1;
    p.ids = block_ids;
    p.out_slots = out_slots;
    p.cache_blocks = g->reserved;
    p.out_rows = n_out_slots;
    p.err = error_word();
    p.block_stride = g->block_stride;
    p.token_stride = g->token_stride;
    p.T = g->block_tokens;
    p.H = g->n_kv_heads;
    p.head_major = head_major;
    return launch_hash(p, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_score_hamming(const uint8_t* codes, int64_t n_slots, int32_t n_kv_heads, int32_t block_tokens, int32_t bits,
                                      const int32_t* req_offsets, const int32_t* slot_ids, const uint8_t* q_codes,
                                      int32_t n_q_heads, int32_t n_req, int32_t total, int32_t cross_head,
                                      int32_t* out_scores, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_req < 0 || total < 0 || n_slots < 0) return UCMX_EPARAM;
    if (n_req == 0 || total == 0) return UCMX_OK;
    if (!codes || !req_offsets || !q_codes || !out_scores) return UCMX_EPARAM;
    if (n_kv_heads < 1 || block_tokens < 1 || bits < 32 || bits % 32 || n_q_heads < 1) return UCMX_EPARAM;
    if (!cross_head && n_q_heads != n_kv_heads) return UCMX_EPARAM;
    if (((uintptr_t)codes & 15) || ((uintptr_t)q_codes & 3)) return UCMX_EPARAM;
    // scores must fit int32: pairs*bits
    if ((long long)n_kv_heads * block_tokens * (cross_head ? n_q_heads : 1) * bits > 0x7fffffffll) return UCMX_EUNSUPPORTED;
    HamParams p{codes, n_slots, error_word(), req_offsets, slot_ids, q_codes, out_scores, n_req, total, n_kv_heads, block_tokens,
                bits / 32, n_q_heads, cross_head ? 1 : 0};
    const int warps_per_cta = kHamThreads / 32;
    int64_t want = ((int64_t)total + warps_per_cta - 1) / warps_per_cta;
    const int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(want > cap ? cap : want);
    if (bits == 128 && n_q_heads <= 15 && !((uintptr_t)q_codes & 15)) {
        if (cross_head) score_hamming_kernel<true><<<grid, kHamThreads, 0, (cudaStream_t)stream>>>(p);
        else score_hamming_kernel<false><<<grid, kHamThreads, 0, (cudaStream_t)stream>>>(p);
    }
    else
        score_hamming_generic_kernel<<<grid, kHamThreads, 0, (cudaStream_t)stream>>>(p);
    UCMX_LAUNCH_CHECK("score_hamming_kernel");
    return UCMX_OK;
}

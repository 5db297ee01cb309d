// Shared device/host helpers for the sm_100a kernels: status plumbing, bf16 bit tricks, and thin
// wrappers over the PTX used for asynchronous bulk copies (cp.async.bulk + mbarrier).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ucmx.h"

namespace ucmx {

constexpr int kSmCountHint = 148;  // B200; the real count is queried once per device

void set_last_error(const char* what, cudaError_t e);
void set_last_text(const char* text);
int32_t* error_word();  // device-visible int that bounded waits report into (NULL if unavailable)
int32_t cuda_status(const char* what, cudaError_t e);
int sm_count();  // multiprocessors of the current device (cached)
bool early_start();  // this thread asked for scoring launches that may begin before the kernel ahead of them ends

// scoring with an explicit error word (NULL: out-of-range ids and lost copies are skipped without a report)
int32_t score_dot_impl(const void* reps, int32_t reps_dtype, int64_t n_slots, int32_t n_kv_heads, int32_t n_rep,
                       int32_t head_dim, const int32_t* req_offsets, const int32_t* slot_ids, const float* q,
                       int32_t n_req, int32_t total, float scale, float* out_scores, const ucmx_peer_exchange* ex,
                       int32_t* err, cudaStream_t st);

// tensor-core (tcgen05) sign-hash encoder; g == NULL: dense vectors, else paged blocks. UCMX_EUNSUPPORTED = not applicable
int32_t hash_encode_tc(const void* x, int64_t n_vec, int64_t x_stride, const ucmx_kv_geometry* g, const int32_t* ids,
                       const int32_t* out_slots, int64_t n_out_rows, int32_t n_blocks, const void* w, int32_t dim, int32_t bits,
                       int32_t head_major, uint8_t* out, cudaStream_t st);

#define UCMX_CUDA(call)                                                  \
    do {                                                                 \
        cudaError_t e__ = (call);                                        \
        if (e__ != cudaSuccess) return ::ucmx::cuda_status(#call, e__);  \
    } while (0)

#define UCMX_LAUNCH_CHECK(name)                                          \
    do {                                                                 \
        cudaError_t e__ = cudaGetLastError();                            \
        if (e__ != cudaSuccess) return ::ucmx::cuda_status(name, e__);   \
    } while (0)

// ------------------------------------------------------------------ bf16 <-> fp32 on raw bits

__device__ __forceinline__ float bf16lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// round-to-nearest-even fp32 -> bf16 bits (NaN stays NaN)
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f)
{
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float bf16_round(float f) { return __uint_as_float(f32_to_bf16_bits(f) << 16); }

// ------------------------------------------------------------------ cache-hinted 16-byte access

__device__ __forceinline__ uint4 ld_stream16(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// plain (coherent) 16-byte load: for memory the GPU does not own exclusively (mapped host memory)
__device__ __forceinline__ uint4 ld_plain16(const void* p)
{
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v)
{
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// ------------------------------------------------------------------ mbarrier + bulk async copy

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// make barrier initialisation visible to the async proxy before the first bulk copy names it
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kSpinLimit polls so that a copy that never lands cannot hang the
// GPU; the caller records the failure and drains. try_wait itself blocks for a hardware-defined
// slice, so the limit is generous (seconds) yet finite.
constexpr uint32_t kSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// global -> shared bulk copy (TMA engine, untiled); completion is signalled on `bar` as bytes.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// The same with an L2 eviction policy: data that is read (or written) once and not again soon is marked
// evict-first, so that a pass over gigabytes does not push the small hot arrays of the next kernels out of L2.
// Programmatic dependent launch.  A kernel launched with the stream-serialization attribute may begin while the
// kernel ahead of it in the stream is still running; early_start_wait() returns once that kernel has finished and its
// writes are visible, early_start_allow() lets the kernel behind this one begin.  Both do nothing in a launch
// without the attribute.
__device__ __forceinline__ void early_start_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void early_start_allow() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint64_t l2_evict_first_policy()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_s2g_hint(void* gdst, const void* smem_src, uint32_t bytes, uint64_t policy)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes), "l"(policy)
                 : "memory");
}
// shared -> global bulk copy, tracked by the issuing thread's bulk async-group
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// order generic-proxy shared-memory writes before async-proxy reads of the same bytes
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ tensor-parallel score exchange
//
// Exchange buffer of one rank (ucmx_peer_exchange in the C ABI; every rank can address every rank's buffer):
//   bytes [0,128)   flag[r]: the last round rank r has delivered into this buffer
//   bytes [128,132) arrival counter of this rank's scoring kernel (thread blocks that are done)
//   bytes [132,136) round counter of this rank (rounds its scoring kernel has completed)
//   bytes [256,..)  inbox[parity][source rank][part_bytes]: partial scores, two halves used alternately
// A round: every rank's scoring kernel stores its partial scores into inbox[round & 1][my_rank] of EVERY rank,
// its last thread block publishes the round number into flag[my_rank] of every rank, and the top-k kernel that
// follows waits for all flags of its own buffer and adds the inbox rows up in rank order.  The round number
// lives in the buffer, not in a kernel argument, so the same launches can be replayed from a CUDA graph.
constexpr int kPeerHeaderBytes = 256;
constexpr int kPeerArriveOffset = 128;
constexpr int kPeerRoundOffset = 132;

// bytes one rank's partial scores take inside a half of the inbox
inline int64_t peer_part_bytes(int64_t n_scores) { return ((n_scores * 4 + 127) / 128) * 128; }

struct PeerPush {
    unsigned char* const* bases;   // device array: base of every rank's exchange buffer, in rank order
    int32_t world, my_rank;
    int64_t part_bytes;            // bytes of one rank's partial scores inside a half (multiple of 128)
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// round this rank's scoring kernel is working on (read by every thread block at its start; the counter moves
// only after all of them have arrived at the end, so they all see the same value)
__device__ __forceinline__ uint32_t peer_round_now(const PeerPush& px)
{
    return *reinterpret_cast<const volatile uint32_t*>(px.bases[px.my_rank] + kPeerRoundOffset) + 1u;
}
__device__ __forceinline__ int64_t peer_inbox_offset(const PeerPush& px, uint32_t round, int src_rank)
{
    return (int64_t)kPeerHeaderBytes + ((int64_t)(round & 1u) * px.world + src_rank) * px.part_bytes;
}
// End of a scoring kernel under tensor parallelism; called by every thread of every thread block after its last
// score store.  The block that arrives last makes the round visible: counter, then one flag per rank.
__device__ __forceinline__ void peer_publish_round(const PeerPush& px, uint32_t round)
{
    __threadfence_system();          // this thread's stores into the peers' inboxes are performed
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned char* mine = px.bases[px.my_rank];
        uint32_t* arrive = reinterpret_cast<uint32_t*>(mine + kPeerArriveOffset);
        const uint32_t blocks = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(arrive, 1u) == blocks - 1u) {
            __threadfence_system();
            *reinterpret_cast<volatile uint32_t*>(arrive) = 0u;
            *reinterpret_cast<volatile uint32_t*>(mine + kPeerRoundOffset) = round;
            for (int t = 0; t < px.world; ++t)
                st_release_sys_u32(reinterpret_cast<uint32_t*>(px.bases[t]) + px.my_rank, round);
        }
    }
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block id of entry i of an id list, and the table row its result goes to.  An id outside the cache (or a row outside
// the table) is never used: the entry is dropped and code 3 is left for ucmx_device_error.  Negative values are the
// documented way to skip an entry and are not reported.
__device__ __forceinline__ int checked_block_id(const int32_t* __restrict__ ids, int64_t i, int64_t n_blocks, int32_t* err)
{
    const int id = __ldg(ids + i);
    if (id >= 0 && (int64_t)id >= n_blocks) {
        if (err) atomicExch(err, 3);
        return -1;
    }
    return id;
}
__device__ __forceinline__ int64_t checked_out_row(const int32_t* __restrict__ out_slots, int64_t i, int64_t n_rows, int32_t* err)
{
    const int64_t row = out_slots ? (int64_t)__ldg(out_slots + i) : i;
    if (row >= 0 && row >= n_rows) {
        if (err) atomicExch(err, 3);
        return -1;
    }
    return row;
}

// lower_bound-style search: the request r with offsets[r] <= c < offsets[r+1]
__device__ __forceinline__ int find_request(const int32_t* __restrict__ offsets, int n_req, int c)
{
    int lo = 0, hi = n_req;  // invariant: offsets[lo] <= c < offsets[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (__ldg(offsets + mid) <= c) lo = mid; else hi = mid;
    }
    return lo;
}

}  // namespace ucmx

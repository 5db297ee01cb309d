// Stage 4: gather / scatter of paged KV block slices between a layer's block pool and a
// contiguous staging area (device memory, or page-locked host memory mapped into the device).
//
// Pure data movement, bound by HBM (device staging: every byte is read once and written once) or
// by the host link (mapped staging).  The device-staging kernel never touches the payload with
// SM instructions: one elected thread per CTA drives a ring of shared-memory stages with bulk
// async copies — global->shared completing on an mbarrier, shared->global tracked by bulk
// async-groups — so the copy engines do the work and the grid is sized to keep every SM's ring
// full.  The mapped-host kernel uses plain 16-byte loads/stores like the reference's
// H2DKernel/D2HKernel (ucm/store/device/cuda/cuda_device.cu:47-69) but with a grid sized to the
// device instead of a fixed 32x256.
#include <cstdlib>

#include "common.cuh"

namespace ucmx {

namespace {

constexpr int kMaxPlanes = 8;

struct XferParams {
    // mode 0: planes + block ids <-> staging;  mode 1: pointer pairs
    int32_t mode;
    int32_t to_staging;  // mode 0: 1 = gather (paged -> staging), 0 = scatter
    unsigned char* planes[kMaxPlanes];
    int32_t n_planes;
    int64_t block_stride;
    const int32_t* ids;
    unsigned char* staging;
    void* const* dst_ptrs;
    const void* const* src_ptrs;
    int64_t n;            // number of blocks (mode 0) or pairs (mode 1)
    int64_t slice_bytes;  // bytes per slice / pair
    int32_t chunk_bytes;
    int32_t chunks_per_slice;
    int64_t items;
    int32_t* err;
};

// Resolve work item -> (src, dst, bytes); bytes == 0 means "skip".
__device__ __forceinline__ void resolve(const XferParams& p, int64_t item, const unsigned char*& src,
                                        unsigned char*& dst, uint32_t& bytes)
{
    const int64_t slice = item / p.chunks_per_slice;
    const int32_t c = (int32_t)(item - slice * p.chunks_per_slice);
    const int64_t off = (int64_t)c * p.chunk_bytes;
    const int64_t left = p.slice_bytes - off;
    bytes = (uint32_t)(left < p.chunk_bytes ? left : p.chunk_bytes);
    if (p.mode == 0) {
        const int64_t i = slice / p.n_planes;
        const int32_t pl = (int32_t)(slice - i * p.n_planes);
        const int32_t id = __ldg(p.ids + i);
        if (id < 0) {
            bytes = 0;
            src = nullptr;
            dst = nullptr;
            return;
        }
        unsigned char* paged = p.planes[pl] + (int64_t)id * p.block_stride + off;
        unsigned char* stag = p.staging + slice * p.slice_bytes + off;
        src = p.to_staging ? paged : stag;
        dst = p.to_staging ? stag : paged;
    } else {
        const unsigned char* s = (const unsigned char*)p.src_ptrs[slice];
        unsigned char* d = (unsigned char*)p.dst_ptrs[slice];
        if (!s || !d || (((uintptr_t)s | (uintptr_t)d) & 15)) {
            if (p.err && (s && d)) atomicExch(p.err, 2);  // misaligned pair: reported, not copied
            bytes = 0;
            src = nullptr;
            dst = nullptr;
            return;
        }
        src = s + off;
        dst = d + off;
    }
}

// Device <-> device: bulk async copies through a shared-memory ring, one driving thread per CTA.
// The driving thread is the only instruction stream, so what it does per chunk is kept short: the work item is
// resolved once (at load time; destination and size wait in shared memory for the store), with 32-bit arithmetic
// when the item count allows, and the block id of the next chunk is requested one chunk ahead, so that its
// latency (an L2 access once the id list outgrows what L1 keeps beside the ring) is not waited for.
template <int STAGES>
__global__ void __launch_bounds__(32) xfer_bulk_kernel(XferParams p)
{
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned char* s_dst[STAGES];
    __shared__ uint32_t s_bytes[STAGES];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    unsigned char* ring = smem + 128;
    if (threadIdx.x != 0) return;

    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();

    const int64_t G = gridDim.x;
    const int64_t first = blockIdx.x;
    if (first >= p.items) return;
    const int64_t my_count = (p.items - first + G - 1) / G;
    const bool ids_mode = p.mode == 0;
    const bool small = p.items < 0x7fffffffll;      // every index fits 32 bits

    // block index (into p.ids) of work item `item`
    auto block_of = [&](int64_t item) -> int64_t {
        if (small) return (int64_t)(((uint32_t)item / (uint32_t)p.chunks_per_slice) / (uint32_t)p.n_planes);
        return (item / p.chunks_per_slice) / p.n_planes;
    };
    int32_t id_ahead = ids_mode ? __ldg(p.ids + block_of(first)) : 0;      // id of the next item to be loaded

    auto load = [&](int64_t j) {
        const int64_t item = first + j * G;
        const int s = (int)(j % STAGES);
        const unsigned char* src = nullptr;
        unsigned char* dst = nullptr;
        uint32_t bytes = 0;
        if (ids_mode) {
            const int32_t id = id_ahead;
            if (j + 1 < my_count) id_ahead = __ldg(p.ids + block_of(item + G));   // used by the next call
            int64_t slice;
            int32_t c;
            if (small) {
                const uint32_t sl = (uint32_t)item / (uint32_t)p.chunks_per_slice;
                c = (int32_t)((uint32_t)item - sl * (uint32_t)p.chunks_per_slice);
                slice = sl;
            } else {
                slice = item / p.chunks_per_slice;
                c = (int32_t)(item - slice * p.chunks_per_slice);
            }
            const int64_t off = (int64_t)c * p.chunk_bytes;
            const int64_t left = p.slice_bytes - off;
            if (id >= 0) {
                bytes = (uint32_t)(left < p.chunk_bytes ? left : p.chunk_bytes);
                const int32_t pl = small ? (int32_t)((uint32_t)slice % (uint32_t)p.n_planes) : (int32_t)(slice % p.n_planes);
                unsigned char* paged = p.planes[pl] + (int64_t)id * p.block_stride + off;
                unsigned char* stag = p.staging + slice * p.slice_bytes + off;
                src = p.to_staging ? paged : stag;
                dst = p.to_staging ? stag : paged;
            }
        } else {
            resolve(p, item, src, dst, bytes);
        }
        s_dst[s] = dst;
        s_bytes[s] = bytes;
        mbar_expect_tx(&full[s], bytes);
        if (bytes) bulk_g2s(ring + (size_t)s * p.chunk_bytes, src, bytes, &full[s]);
    };

    const int64_t pre = my_count < STAGES ? my_count : STAGES;
    for (int64_t j = 0; j < pre; ++j) load(j);

    bool failed = false;
    for (int64_t j = 0; j < my_count; ++j) {
        const int s = (int)(j % STAGES);
        const uint32_t parity = (uint32_t)(j / STAGES) & 1u;
        if (!mbar_wait(&full[s], parity)) {
            failed = true;
            if (p.err) atomicExch(p.err, 1);
            break;
        }
        const uint32_t bytes = s_bytes[s];
        if (bytes) bulk_s2g(s_dst[s], ring + (size_t)s * p.chunk_bytes, bytes);
        bulk_commit();
        // refill the stage whose store was committed one group ago
        if (j >= 1 && j - 1 + STAGES < my_count) {
            bulk_wait_read<1>();
            load(j - 1 + STAGES);
        }
    }
    bulk_wait_all<0>();
    if (failed) {
        // loads may still be landing in this CTA's shared memory: bounded wait on every stage
        for (int s = 0; s < STAGES; ++s) {
            (void)mbar_wait(&full[s], 0);
            (void)mbar_wait(&full[s], 1);
        }
    }
}

// Any address space the GPU can reach (device, mapped host): 16-byte loads and stores.
// A warp moves 512 contiguous bytes per step; four steps are kept in flight.
__global__ void __launch_bounds__(256) xfer_plain_kernel(XferParams p)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    for (int64_t item = w; item < p.items; item += warps) {
        const unsigned char* src;
        unsigned char* dst;
        uint32_t bytes;
        resolve(p, item, src, dst, bytes);
        if (!bytes) continue;
        const uint32_t n16 = bytes >> 4;
        uint32_t i = lane;
        for (; i + 96 < n16; i += 128) {
            const uint4 a = ld_plain16(src + (size_t)i * 16);
            const uint4 b = ld_plain16(src + (size_t)(i + 32) * 16);
            const uint4 c = ld_plain16(src + (size_t)(i + 64) * 16);
            const uint4 d = ld_plain16(src + (size_t)(i + 96) * 16);
            *reinterpret_cast<uint4*>(dst + (size_t)i * 16) = a;
            *reinterpret_cast<uint4*>(dst + (size_t)(i + 32) * 16) = b;
            *reinterpret_cast<uint4*>(dst + (size_t)(i + 64) * 16) = c;
            *reinterpret_cast<uint4*>(dst + (size_t)(i + 96) * 16) = d;
        }
        for (; i < n16; i += 32) *reinterpret_cast<uint4*>(dst + (size_t)i * 16) = ld_plain16(src + (size_t)i * 16);
    }
}

int32_t launch_xfer(XferParams& p, bool host_memory, cudaStream_t st)
{
    p.err = error_word();
    const int sms = sm_count();
    if (host_memory) {
        p.chunk_bytes = 4096;
        p.chunks_per_slice = (int32_t)((p.slice_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
        p.items = p.n * (p.mode == 0 ? p.n_planes : 1) * p.chunks_per_slice;
        int64_t want = (p.items + 7) / 8;
        int grid = (int)(want > (int64_t)sms * 4 ? (int64_t)sms * 4 : want);
        xfer_plain_kernel<<<grid, 256, 0, st>>>(p);
        UCMX_LAUNCH_CHECK("xfer_plain_kernel");
        return UCMX_OK;
    }
    // tuning knobs (read once): chunk size, ring depth, CTAs per SM.  Measured defaults: the same 24 chunks of 8 KiB
    // in flight per SM either way, as two CTAs with rings of twelve for slices of 128 KiB and more (256 KiB: 6.7 TB/s
    // against 6.0) and as three CTAs with rings of eight for smaller ones (32 KiB: 6.5 TB/s against 6.1; 64 KiB:
    // 6.7 against 6.4).
    static const int k_chunk = [] { const char* e = getenv("UCMX_XFER_CHUNK"); const int v = e ? atoi(e) : 0; return (v >= 1024 && v <= 65536 && v % 16 == 0) ? v : 8192; }();
    static const int env_stages = [] { const char* e = getenv("UCMX_XFER_STAGES"); const int v = e ? atoi(e) : 0; return (v == 2 || v == 3 || v == 4 || v == 6 || v == 8 || v == 12 || v == 16) ? v : 0; }();
    static const int env_per_sm = [] { const char* e = getenv("UCMX_XFER_CTAS_PER_SM"); const int v = e ? atoi(e) : 0; return (v >= 1 && v <= 16) ? v : 0; }();
    static const int64_t k_large = [] { const char* e = getenv("UCMX_XFER_LARGE_SLICE"); const long long v = e ? atoll(e) : 0; return v > 0 ? (int64_t)v : (int64_t)131072; }();
    const bool large = p.slice_bytes >= k_large;
    const int k_stages = env_stages ? env_stages : (large ? 12 : 8);
    const int k_per_sm = env_per_sm ? env_per_sm : (large ? 2 : 3);
    p.chunk_bytes = k_chunk;
    if (p.slice_bytes < p.chunk_bytes) p.chunk_bytes = (int32_t)p.slice_bytes;
    p.chunks_per_slice = (int32_t)((p.slice_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
    p.items = p.n * (p.mode == 0 ? p.n_planes : 1) * p.chunks_per_slice;
    const size_t smem = 128 + (size_t)k_stages * p.chunk_bytes;
    if (smem > 220 * 1024) return UCMX_EUNSUPPORTED;
    void (*kern)(XferParams) = xfer_bulk_kernel<8>;
    switch (k_stages) {
        case 4: kern = xfer_bulk_kernel<4>; break;
        case 2: kern = xfer_bulk_kernel<2>; break;
        case 3: kern = xfer_bulk_kernel<3>; break;
        case 6: kern = xfer_bulk_kernel<6>; break;
        case 12: kern = xfer_bulk_kernel<12>; break;
        case 16: kern = xfer_bulk_kernel<16>; break;
        default: break;
    }
    UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int ctas_per_sm = k_per_sm;
    while (ctas_per_sm > 1 && (size_t)ctas_per_sm * (smem + 1024) > 227 * 1024) --ctas_per_sm;
    int64_t grid = (int64_t)sms * ctas_per_sm;
    if (grid > p.items) grid = p.items;
    kern<<<(unsigned)grid, 32, smem, st>>>(p);
    UCMX_LAUNCH_CHECK("xfer_bulk_kernel");
    return UCMX_OK;
}

int32_t blocks_common(void* const* planes, int32_t n_planes, int64_t block_stride_bytes, const int32_t* block_ids,
                      int32_t n, int64_t slice_bytes, void* staging, int32_t staging_is_host, int to_staging,
                      cudaStream_t st)
{
    if (n < 0 || n_planes < 1 || n_planes > kMaxPlanes) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (!planes || !block_ids || !staging) return UCMX_EPARAM;
    if (slice_bytes <= 0 || (slice_bytes & 15) || (block_stride_bytes & 15) || ((uintptr_t)staging & 15))
        return UCMX_EPARAM;
    XferParams p{};
    p.mode = 0;
    p.to_staging = to_staging;
    for (int i = 0; i < n_planes; ++i) {
        if (!planes[i] || ((uintptr_t)planes[i] & 15)) return UCMX_EPARAM;
        p.planes[i] = (unsigned char*)planes[i];
    }
    p.n_planes = n_planes;
    p.block_stride = block_stride_bytes;
    p.ids = block_ids;
    p.staging = (unsigned char*)staging;
    p.n = n;
    p.slice_bytes = slice_bytes;
    return launch_xfer(p, staging_is_host != 0, st);
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_gather_blocks(const void* const* planes, int32_t n_planes, int64_t block_stride_bytes,
                                      const int32_t* block_ids, int32_t n, int64_t slice_bytes, void* staging,
                                      int32_t staging_is_host, ucmx_stream_t stream)
{
    return ucmx::blocks_common((void* const*)planes, n_planes, block_stride_bytes, block_ids, n, slice_bytes,
                               staging, staging_is_host, 1, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_scatter_blocks(void* const* planes, int32_t n_planes, int64_t block_stride_bytes,
                                       const int32_t* block_ids, int32_t n, int64_t slice_bytes,
                                       const void* staging, int32_t staging_is_host, ucmx_stream_t stream)
{
    return ucmx::blocks_common(planes, n_planes, block_stride_bytes, block_ids, n, slice_bytes, (void*)staging,
                               staging_is_host, 0, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_copy_batch(void* const* dst_ptrs, const void* const* src_ptrs, int32_t number,
                                   int64_t count, int32_t any_host_memory, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (number < 0) return UCMX_EPARAM;
    if (number == 0 || count == 0) return UCMX_OK;
    if (!dst_ptrs || !src_ptrs || count < 0 || (count & 15)) return UCMX_EPARAM;
    XferParams p{};
    p.mode = 1;
    p.dst_ptrs = dst_ptrs;
    p.src_ptrs = src_ptrs;
    p.n = number;
    p.slice_bytes = count;
    return launch_xfer(p, any_host_memory != 0, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_memcpy_async(void* dst, const void* src, int64_t bytes, ucmx_stream_t stream)
{
    if (bytes < 0) return UCMX_EPARAM;
    if (bytes == 0) return UCMX_OK;
    if (!dst || !src) return UCMX_EPARAM;
    UCMX_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    return UCMX_OK;
}

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
    // mode 0: planes + block ids <-> staging;  mode 1: pointer pairs;  mode 2: planes + ids -> other planes + ids
    int32_t mode;
    int32_t to_staging;  // mode 0: 1 = gather (paged -> staging), 0 = scatter
    unsigned char* planes[kMaxPlanes];
    int32_t n_planes;
    int64_t block_stride;
    const int32_t* ids;
    int64_t n_blocks;     // blocks a plane holds: an id at or beyond it is skipped and reported
    unsigned char* dst_planes[kMaxPlanes];   // mode 2
    int64_t dst_block_stride;
    const int32_t* dst_ids;
    int64_t n_dst_blocks;
    const int32_t* n_dev;  // mode 2, optional: entries to process, read on the device (then cleared by the kernel)
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
        if (id < 0 || (int64_t)id >= p.n_blocks) {
            if (id >= 0 && p.err) atomicExch(p.err, 3);   // outside the cache: reported, not touched
            bytes = 0;
            src = nullptr;
            dst = nullptr;
            return;
        }
        unsigned char* paged = p.planes[pl] + (int64_t)id * p.block_stride + off;
        unsigned char* stag = p.staging + slice * p.slice_bytes + off;
        src = p.to_staging ? paged : stag;
        dst = p.to_staging ? stag : paged;
    } else if (p.mode == 2) {
        const int64_t i = slice / p.n_planes;
        const int32_t pl = (int32_t)(slice - i * p.n_planes);
        const int32_t sid = __ldg(p.ids + i), did = __ldg(p.dst_ids + i);
        if (sid < 0 || did < 0 || (int64_t)sid >= p.n_blocks || (int64_t)did >= p.n_dst_blocks) {
            if (sid >= 0 && did >= 0 && p.err) atomicExch(p.err, 3);
            bytes = 0;
            src = nullptr;
            dst = nullptr;
            return;
        }
        src = p.planes[pl] + (int64_t)sid * p.block_stride + off;
        dst = p.dst_planes[pl] + (int64_t)did * p.dst_block_stride + off;
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
__device__ __forceinline__ void xfer_bulk_body(const XferParams& p, const int64_t items)
{
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned char* s_dst[STAGES];
    __shared__ uint32_t s_bytes[STAGES];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    unsigned char* ring = smem + 128;
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
    // every byte passes through L2 exactly once in each direction: evict-first keeps what the neighbouring kernels
    // of a decode step reuse (block tables, offsets, queries, scores) resident across a gather of gigabytes
    const uint64_t stream_once = l2_evict_first_policy();

    const int64_t G = gridDim.x;
    const int64_t first = blockIdx.x;
    if (first >= items) return;
    const int64_t my_count = (items - first + G - 1) / G;
    const bool ids_mode = p.mode == 0;
    const bool small = items < 0x7fffffffll;      // every index fits 32 bits

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
            if (id >= 0 && (int64_t)id >= p.n_blocks) {
                if (p.err) atomicExch(p.err, 3);           // outside the cache: reported, not touched
            } else if (id >= 0) {
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
        if (bytes) bulk_g2s_hint(ring + (size_t)s * p.chunk_bytes, src, bytes, &full[s], stream_once);
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
        if (bytes) bulk_s2g_hint(s_dst[s], ring + (size_t)s * p.chunk_bytes, bytes, stream_once);
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

template <int STAGES>
__global__ void __launch_bounds__(32) xfer_bulk_kernel(XferParams p)
{
    if (threadIdx.x != 0) return;
    int64_t items = p.items;
    if (p.n_dev) {
        // the number of entries is known on the device only (the load list a remap round left behind)
        int64_t n = *reinterpret_cast<const volatile int32_t*>(p.n_dev);
        n = n < 0 ? 0 : (n > p.n ? p.n : n);
        items = n * p.n_planes * p.chunks_per_slice;
    }
    xfer_bulk_body<STAGES>(p, items);
    if (p.n_dev) {
        // every thread block has read the count by now; the last one to finish clears it (and the arrival word
        // beside it) for the next round
        __threadfence();
        unsigned* arrive = reinterpret_cast<unsigned*>(const_cast<int32_t*>(p.n_dev)) + 1;
        if (atomicAdd(arrive, 1u) == gridDim.x - 1) {
            *reinterpret_cast<volatile int32_t*>(const_cast<int32_t*>(p.n_dev)) = 0;
            *reinterpret_cast<volatile unsigned*>(arrive) = 0u;
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
        p.items = p.n * (p.mode == 1 ? 1 : p.n_planes) * p.chunks_per_slice;
        int64_t want = (p.items + 7) / 8;
        int grid = (int)(want > (int64_t)sms * 4 ? (int64_t)sms * 4 : want);
        xfer_plain_kernel<<<grid, 256, 0, st>>>(p);
        UCMX_LAUNCH_CHECK("xfer_plain_kernel");
        return UCMX_OK;
    }
    // Two thread blocks per SM with rings of seven 8 KiB chunks.  Alone, a gather runs as fast with anything from 2 x 5
    // to 2 x 12 chunks per SM (6.5-6.6 TB/s for slices of 64 and 256 KiB, 6.1-6.3 for 32 KiB), and three blocks of eight
    // are a little faster still for 64 KiB slices; inside a decode step the small footprint wins by far, because it
    // leaves more than half of an SM's shared memory to the scoring and top-k kernels of the next layer, which then
    // run beside the gather instead of between two gathers (measured per layer, next layer's selection on a second
    // stream: 32 KiB slices 334 us against 369 with 3 x 8; 64 KiB 664 against 724; 256 KiB 9.79 ms per 32-layer step
    // against 9.91 with 2 x 12).  Four chunks per block are too few (10.4 ms).
    constexpr int k_chunk = 8192;
    constexpr int k_stages = 7;
    constexpr int k_per_sm = 2;
    p.chunk_bytes = k_chunk;
    if (p.slice_bytes < p.chunk_bytes) p.chunk_bytes = (int32_t)p.slice_bytes;
    p.chunks_per_slice = (int32_t)((p.slice_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
    p.items = p.n * (p.mode == 1 ? 1 : p.n_planes) * p.chunks_per_slice;
    const size_t smem = 128 + (size_t)k_stages * p.chunk_bytes;
    if (smem > 220 * 1024) return UCMX_EUNSUPPORTED;
    void (*kern)(XferParams) = xfer_bulk_kernel<k_stages>;
    {
        static int smem_set[64];                  // per device: dynamic shared memory limit already raised to this
        int dev = 0;
        UCMX_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || smem_set[dev] < (int)smem) {
            UCMX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (dev >= 0 && dev < 64) smem_set[dev] = (int)smem;
        }
    }
    int ctas_per_sm = k_per_sm;
    while (ctas_per_sm > 1 && (size_t)ctas_per_sm * (smem + 1024) > 227 * 1024) --ctas_per_sm;
    int64_t grid = (int64_t)sms * ctas_per_sm;
    if (grid > p.items) grid = p.items;
    kern<<<(unsigned)grid, 32, smem, st>>>(p);
    UCMX_LAUNCH_CHECK("xfer_bulk_kernel");
    return UCMX_OK;
}

int32_t blocks_common(void* const* planes, int32_t n_planes, int64_t block_stride_bytes, int64_t n_blocks,
                      const int32_t* block_ids, int32_t n, int64_t slice_bytes, void* staging, int32_t staging_is_host,
                      int to_staging, cudaStream_t st)
{
    if (n < 0 || n_planes < 1 || n_planes > kMaxPlanes || n_blocks < 1) return UCMX_EPARAM;
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
    p.n_blocks = n_blocks;
    p.staging = (unsigned char*)staging;
    p.n = n;
    p.slice_bytes = slice_bytes;
    return launch_xfer(p, staging_is_host != 0, st);
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_gather_blocks(const void* const* planes, int32_t n_planes, int64_t block_stride_bytes,
                                      int64_t n_blocks, const int32_t* block_ids, int32_t n, int64_t slice_bytes,
                                      void* staging, int32_t staging_is_host, ucmx_stream_t stream)
{
    return ucmx::blocks_common((void* const*)planes, n_planes, block_stride_bytes, n_blocks, block_ids, n, slice_bytes,
                               staging, staging_is_host, 1, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_scatter_blocks(void* const* planes, int32_t n_planes, int64_t block_stride_bytes,
                                       int64_t n_blocks, const int32_t* block_ids, int32_t n, int64_t slice_bytes,
                                       const void* staging, int32_t staging_is_host, ucmx_stream_t stream)
{
    return ucmx::blocks_common(planes, n_planes, block_stride_bytes, n_blocks, block_ids, n, slice_bytes, (void*)staging,
                               staging_is_host, 0, (cudaStream_t)stream);
}

extern "C" int32_t ucmx_move_blocks(const void* const* src_planes, void* const* dst_planes, int32_t n_planes,
                                    int64_t src_block_stride_bytes, int64_t n_src_blocks, const int32_t* src_ids,
                                    int64_t dst_block_stride_bytes, int64_t n_dst_blocks, const int32_t* dst_ids,
                                    int32_t n, const int32_t* n_device, int64_t slice_bytes, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n < 0 || n_planes < 1 || n_planes > kMaxPlanes || n_src_blocks < 1 || n_dst_blocks < 1) return UCMX_EPARAM;
    if (n == 0) return UCMX_OK;
    if (!src_planes || !dst_planes || !src_ids || !dst_ids) return UCMX_EPARAM;
    if (slice_bytes <= 0 || (slice_bytes & 15) || (src_block_stride_bytes & 15) || (dst_block_stride_bytes & 15)) return UCMX_EPARAM;
    XferParams p{};
    p.mode = 2;
    for (int i = 0; i < n_planes; ++i) {
        if (!src_planes[i] || !dst_planes[i] || (((uintptr_t)src_planes[i] | (uintptr_t)dst_planes[i]) & 15)) return UCMX_EPARAM;
        p.planes[i] = (unsigned char*)src_planes[i];
        p.dst_planes[i] = (unsigned char*)dst_planes[i];
    }
    p.n_planes = n_planes;
    p.block_stride = src_block_stride_bytes;
    p.ids = src_ids;
    p.n_blocks = n_src_blocks;
    p.dst_block_stride = dst_block_stride_bytes;
    p.dst_ids = dst_ids;
    p.n_dst_blocks = n_dst_blocks;
    p.n_dev = n_device;
    p.n = n;
    p.slice_bytes = slice_bytes;
    return launch_xfer(p, false, (cudaStream_t)stream);
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

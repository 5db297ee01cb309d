// Stage 3 -> 4 glue: which HBM block serves each selected logical block, and what has to be loaded.
//
// The reference keeps, per request and layer, two std::map's (logical block -> HBM block and back)
// plus a free list, and walks them on CPU threads for every decode step
// (GSAPrefetchEngineC::GetHitAndMissBlock / RunPrefetchH2D / RunOneBsPrefetch / LoadKVToHBM,
// ucm/sparse/gsa/prefetch/src/kvcache_pre.cpp:206-322); ESA does the same job with Python sets
// (ucm/sparse/esa/esa.py:313-334).  Here the state is three flat arrays per request (the HBM
// blocks it owns in ascending physical order, the logical block each holds, a free flag) and one
// thread block per request replays a round: hits stay where they are, misses take free slots in
// order, the block table and the load list come out, the state is updated in place - so the
// selected ids never have to visit the host between top-k and the block transfer.
#include "common.cuh"

namespace ucmx {
namespace {

struct RemapParams {
    int32_t* slot_logical;
    uint8_t* slot_free;
    const int32_t* slot_phys;
    const int32_t* slot_offsets;
    const int32_t* sel;
    const int32_t* sel_offsets;
    const int32_t* sel_counts;  // optional: valid entries of each request's selection
    int32_t max_logical;
    int32_t max_slots;          // slots per request the shared-memory lists were sized for
    int32_t* table;
    int32_t* load_logical;
    int32_t* load_phys;
    int32_t* load_counts;
    ucmx_remap_moves mv;             // optional (mv.move_count != NULL): one packed move list for all requests
    int32_t* err;
};

constexpr int kRemapThreads = 256;

// exclusive prefix of a flag over the block in thread order; `total` gets the block sum
__device__ __forceinline__ int excl_scan(bool flag, int* s_warp, int& total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = kRemapThreads / 32;
    const unsigned b = __ballot_sync(0xffffffffu, flag);
    const int in_warp = __popc(b & ((1u << lane) - 1u));
    if (lane == 0) s_warp[warp] = __popc(b);
    __syncthreads();
    int before = 0, tot = 0;
    for (int w = 0; w < nwarp; ++w) {
        const int v = s_warp[w];
        if (w < warp) before += v;
        tot += v;
    }
    __syncthreads();
    total = tot;
    return before + in_warp;
}

__global__ void __launch_bounds__(kRemapThreads) remap_resident_kernel(RemapParams p)
{
    extern __shared__ __align__(16) int32_t sm[];
    int32_t* lookup = sm;  // logical block -> slot (local index) or -1, max_logical entries
    __shared__ int s_warp[32];

    const int r = blockIdx.x, tid = threadIdx.x;
    const int s0 = __ldg(p.slot_offsets + r), n_slots = __ldg(p.slot_offsets + r + 1) - s0;
    const int j0 = __ldg(p.sel_offsets + r);
    int n_sel = __ldg(p.sel_offsets + r + 1) - j0;
    if (p.sel_counts) {
        const int c = __ldg(p.sel_counts + r);
        if (c < 0) return;                          // a negative count: this request sits the round out, state untouched
        n_sel = min(n_sel, c);
    }
    int32_t* slot_logical = p.slot_logical + s0;
    uint8_t* slot_free = p.slot_free + s0;
    const int32_t* slot_phys = p.slot_phys + s0;
    const int32_t* sel = p.sel + j0;
    int32_t* table = p.table + j0;
    // free slots in order, then the hit flags, live in shared memory behind the lookup table
    int32_t* free_list = lookup + p.max_logical;       // n_slots entries
    int32_t* hit = free_list + n_slots;                // n_slots entries

    if (n_slots > p.max_slots || n_slots < 0) {
        // more slots than the lists behind the lookup table were sized for: refuse the request, touch nothing
        for (int j = tid; j < n_sel; j += kRemapThreads) table[j] = -1;
        const int room = __ldg(p.sel_offsets + r + 1) - j0;
        for (int j = tid; j < room; j += kRemapThreads) {
            p.load_logical[j0 + j] = -1;
            p.load_phys[j0 + j] = -1;
        }
        if (tid == 0) {
            p.load_counts[r] = 0;
            if (p.err) atomicExch(p.err, 3);
        }
        return;
    }
    for (int i = tid; i < p.max_logical; i += kRemapThreads) lookup[i] = -1;
    for (int i = tid; i < n_slots; i += kRemapThreads) hit[i] = 0;
    __syncthreads();
    for (int s = tid; s < n_slots; s += kRemapThreads) {
        const int l = slot_logical[s];
        if (l >= 0 && l < p.max_logical) lookup[l] = s;
        else if (l >= p.max_logical && p.err) atomicExch(p.err, 3);  // state outside the declared range
    }
    __syncthreads();

    // hits: resident selected blocks keep their slot
    for (int j = tid; j < n_sel; j += kRemapThreads) {
        const int l = sel[j];
        int out = -1;
        if (l >= 0 && l < p.max_logical) {
            const int s = lookup[l];
            if (s >= 0) {
                hit[s] = 1;
                out = __ldg(slot_phys + s);
            }
        }
        table[j] = out;
    }
    __syncthreads();

    // free list of this round: listed free by the previous round and not hit now, in slot order
    int n_free = 0;
    for (int c0 = 0; c0 < n_slots; c0 += kRemapThreads) {
        const int s = c0 + tid;
        const bool f = s < n_slots && slot_free[s] != 0 && hit[s] == 0 && __ldg(slot_phys + s) >= 0;
        int tot;
        const int pos = n_free + excl_scan(f, s_warp, tot);
        if (f) free_list[pos] = s;
        n_free += tot;
    }
    __syncthreads();

    // misses in selection order take the free slots in list order
    int n_miss = 0;
    for (int c0 = 0; c0 < n_sel; c0 += kRemapThreads) {
        const int j = c0 + tid;
        const bool m = j < n_sel && table[j] == -1 && sel[j] >= 0 && sel[j] < p.max_logical;
        int tot;
        const int pos = n_miss + excl_scan(m, s_warp, tot);
        if (m && pos < n_free) {
            const int s = free_list[pos];
            const int phys = __ldg(slot_phys + s);
            slot_logical[s] = sel[j];
            hit[s] = 1;
            table[j] = phys;
            p.load_logical[j0 + pos] = sel[j];
            p.load_phys[j0 + pos] = phys;
        }
        n_miss += tot;
    }
    __syncthreads();
    for (int s = tid; s < n_slots; s += kRemapThreads) slot_free[s] = (hit[s] || __ldg(slot_phys + s) < 0) ? 0 : 1;
    // the rest of this request's room in the load lists is marked empty, so that a block mover can take the lists
    // of all requests as one array and skip what is not a load
    const int n_load = min(n_miss, n_free);
    const int room = __ldg(p.sel_offsets + r + 1) - j0;
    for (int j = n_load + tid; j < room; j += kRemapThreads) {
        p.load_logical[j0 + j] = -1;
        p.load_phys[j0 + j] = -1;
    }
    if (tid == 0) p.load_counts[r] = n_load;
    if (p.mv.move_count && n_load > 0) {
        // this request's loads join the list of moves of the whole batch
        __shared__ int s_base;
        if (tid == 0) s_base = atomicAdd(p.mv.move_count, n_load);
        __syncthreads();
        const int src0 = p.mv.src_map_offsets ? __ldg(p.mv.src_map_offsets + r) : 0;
        for (int j = tid; j < n_load; j += kRemapThreads) {
            p.mv.move_src[s_base + j] = __ldg(p.mv.src_map + src0 + p.load_logical[j0 + j]);
            p.mv.move_dst[s_base + j] = p.load_phys[j0 + j];
        }
    }
}

}  // namespace
}  // namespace ucmx

extern "C" int32_t ucmx_remap_resident(int32_t* slot_logical, uint8_t* slot_free, const int32_t* slot_phys,
                                       const int32_t* slot_offsets, const int32_t* sel, const int32_t* sel_offsets,
                                       const int32_t* sel_counts, int32_t n_req, int32_t max_logical,
                                       int32_t max_slots, int32_t* table, int32_t* load_logical, int32_t* load_phys,
                                       int32_t* load_counts, const ucmx_remap_moves* moves, ucmx_stream_t stream)
{
    using namespace ucmx;
    if (n_req < 0 || max_logical < 1 || max_slots < 0) return UCMX_EPARAM;
    if (n_req == 0) return UCMX_OK;
    if (!slot_logical || !slot_free || !slot_phys || !slot_offsets || !sel || !sel_offsets || !table || !load_logical ||
        !load_phys || !load_counts)
        return UCMX_EPARAM;
    ucmx_remap_moves mv{};
    if (moves) {
        if (!moves->src_map || !moves->move_src || !moves->move_dst || !moves->move_count) return UCMX_EPARAM;
        mv = *moves;
    }
    const size_t smem = ((size_t)max_logical + 2 * (size_t)max_slots) * sizeof(int32_t);
    if (smem > 200 * 1024) return UCMX_EUNSUPPORTED;
    if (smem > 48 * 1024)
        UCMX_CUDA(cudaFuncSetAttribute(remap_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    RemapParams p{slot_logical, slot_free, slot_phys, slot_offsets, sel, sel_offsets, sel_counts, max_logical,
                  max_slots, table, load_logical, load_phys, load_counts, mv, error_word()};
    remap_resident_kernel<<<n_req, kRemapThreads, smem, (cudaStream_t)stream>>>(p);
    UCMX_LAUNCH_CHECK("remap_resident_kernel");
    return UCMX_OK;
}

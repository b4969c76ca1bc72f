// Stage (b) and (d): from per-splat tile counts to the list of (tile, splat) pairs, and from the sorted
// list to per-tile ranges.
//
// The reference emits one 64-bit (tile | depth) key per pair in splat-id order and sorts all 64 bits
// (cpp/rasterizer_torch.cu:83-113, cpp/rasterizer_kernels.cu:252-306).  Here the splats are first put
// in (depth, id) order -- a sort over N items instead of K >> N -- and the pairs are emitted in that
// order, so the big list only needs a stable sort on its tile bits afterwards.  The result is the same
// list the reference's full-key sort produces: within a tile, ascending depth bits, ties by id.
//
//   plan:   sort depth keys  ->  scan tile counts in that order (single pass, decoupled look-back)
//   emit:   each warp expands its 32 splats' rectangles into consecutive packed pairs
//   ranges: one binary search per tile over the sorted list (replaces mark + max-scan, :23-42)
#include "common.cuh"

namespace dsb {

namespace {

constexpr int kScanThreads = 1024;
constexpr u64 kScanAggregate = 1ull << 62;
constexpr u64 kScanInclusive = 1ull << 63;
constexpr u64 kScanValue = (1ull << 62) - 1;

struct PlanTail {       // lives after the sort workspace
    u64 total;
    u32 tile_counter;
    int status;
};

// Single-pass exclusive scan of tiles_touched taken in depth order.
__global__ void __launch_bounds__(kScanThreads)
scan_counts_kernel(const u64* __restrict__ depth_keys_sorted, const int32_t* __restrict__ tiles, const int n,
                   const int drop_last, u32* __restrict__ offsets, u64* __restrict__ lookback, PlanTail* __restrict__ tail) {
    __shared__ u32 s_wsum[32];
    __shared__ u32 s_tile;
    __shared__ u64 s_prefix;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tile = atomicAdd(&tail->tile_counter, 1u);
    __syncthreads();
    const u32 tile = s_tile;
    const int j = (int)tile * kScanThreads + tid;
    u32 c = 0;
    if (j < n) {
        const u32 id = (u32)depth_keys_sorted[j];
        c = (u32)tiles[id];
        if (drop_last && id == (u32)(n - 1)) c = 0;  // the reference never emits pairs for the last splat
    }
    u32 incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        u32 w = s_wsum[lane];
        u32 wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += t;
        }
        s_wsum[lane] = wi - w;  // exclusive prefix of the warps
        if (lane == 31) {
            const u64 block_total = wi;
            volatile u64* mine = lookback + tile;
            u64 earlier = 0;
            if (tile == 0) {
                *mine = block_total | kScanInclusive;
            } else {
                *mine = block_total | kScanAggregate;
                int p = (int)tile - 1;
                u32 polls = 0;
                while (p >= 0) {
                    const u64 v = *(volatile const u64*)(lookback + p);
                    if ((v >> 62) == 0) {
                        if (++polls > kSpinLimit) { atomicExch(&tail->status, DSB_ERR_DEVICE_WAIT_EXPIRED); break; }
                        __nanosleep(40);
                        continue;
                    }
                    earlier += v & kScanValue;
                    if (v & kScanInclusive) break;
                    --p;
                }
                *mine = ((earlier + block_total) & kScanValue) | kScanInclusive;
            }
            s_prefix = earlier;
            if ((int)tile == (n + kScanThreads - 1) / kScanThreads - 1) tail->total = earlier + block_total;
        }
    }
    __syncthreads();
    if (j < n) {
        const u64 off = s_prefix + s_wsum[warp] + (incl - c);
        offsets[j] = off > 0xffffffffull ? 0xffffffffu : (u32)off;
    }
}

// One warp per 32 depth-ordered splats: their pair ranges are consecutive, so the warp walks the
// concatenated range 32 positions at a time; each lane finds the owning splat by a 5-step search over
// the lanes' running counts and writes one packed pair.  All stores are consecutive 8-byte lanes.
// With HIST the kernel also counts the digits the following tile sort will look at (it knows every tile id
// it writes), which spares that sort a pass over the list.
template <bool HIST>
__global__ void __launch_bounds__(256)
emit_pairs_kernel(const int n, const u32 k, const int tiles_x, const int drop_last, const float4* __restrict__ records,
                  const int32_t* __restrict__ tiles, const u64* __restrict__ depth_keys_sorted,
                  const u32* __restrict__ offsets, u64* __restrict__ pairs, const SortPlan plan, u32* __restrict__ hist) {
    __shared__ u32 s_hist[HIST ? 4 : 1][256];
    if (HIST) {
        for (int i = threadIdx.x; i < plan.npass * 256; i += 256) (&s_hist[0][0])[i] = 0;
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;  // position in depth order; warps are aligned to 32
    u32 id = 0, c = 0, off = 0;
    int x0 = 0, y0 = 0, w = 1;
    if (j < n) {
        id = (u32)depth_keys_sorted[j];
        c = (u32)tiles[id];
        if (drop_last && id == (u32)(n - 1)) c = 0;
        off = offsets[j];
        if (c) {
            const float4 q2 = __ldg(records + (size_t)id * 3 + 2);
            const u32 rx = __float_as_uint(q2.z), ry = __float_as_uint(q2.w);
            x0 = (int)(rx & 0xffffu);
            w = (int)(rx >> 16) - x0;
            y0 = (int)(ry & 0xffffu);
        }
    }
    u32 incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    const u32 excl = incl - c;
    const u32 total = __shfl_sync(0xffffffffu, incl, 31);
    const u32 warp_base = __shfl_sync(0xffffffffu, off, 0);
    for (u32 base = 0; base < total; base += 32) {
        const u32 p = base + lane;
        // owner = number of lanes whose inclusive count is <= p
        int owner = 0;
#pragma unroll
        for (int step = 16; step >= 1; step >>= 1) {
            const u32 t = __shfl_sync(0xffffffffu, incl, owner + step - 1);
            if (t <= p) owner += step;
        }
        owner = min(owner, 31);
        const u32 o_excl = __shfl_sync(0xffffffffu, excl, owner);
        const u32 o_id = __shfl_sync(0xffffffffu, id, owner);
        const int o_x0 = __shfl_sync(0xffffffffu, x0, owner);
        const int o_y0 = __shfl_sync(0xffffffffu, y0, owner);
        const int o_w = __shfl_sync(0xffffffffu, w, owner);
        u64 pair = 0;
        bool wrote = false;
        if (p < total) {
            const u32 r = p - o_excl;
            const u32 ry = r / (u32)o_w;
            const u32 tile = (u32)(o_y0 + (int)ry) * (u32)tiles_x + (u32)o_x0 + (r - ry * (u32)o_w);
            const u32 dst = warp_base + p;
            pair = ((u64)tile << 32) | o_id;
            wrote = dst < k;
            if (wrote) pairs[dst] = pair;
        }
        if (HIST) {
            // Lowest digit: consecutive lanes hold consecutive tile ids, so the counters rarely collide.
            if (wrote) atomicAdd(&s_hist[0][sort_digit(pair, plan.shift[0], plan.mask[0], plan.flip[0])], 1u);
            // Higher digits are nearly constant inside a warp: one atomic per group of equal digits.
            for (int q = 1; q < plan.npass; ++q) {
                const u32 d = sort_digit(pair, plan.shift[q], plan.mask[q], plan.flip[q]);
                const u32 m = warp_peers(d, wrote, plan.bits[q]);
                if (wrote && (m & ((1u << lane) - 1u)) == 0) atomicAdd(&s_hist[q][d], (u32)__popc(m));
            }
        }
    }
    if (HIST) {
        __syncthreads();
        for (int i = threadIdx.x; i < plan.npass * 256; i += 256) {
            const u32 c = (&s_hist[0][0])[i];
            if (c) atomicAdd(hist + i, c);
        }
    }
}

// ranges[t] = number of sorted items whose tile id (high 32 bits, signed) is < t, t = 0..T.
__global__ void tile_ranges_kernel(const u64* __restrict__ sorted, const u32 k, const int num_tiles,
                                   int32_t* __restrict__ ranges) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > num_tiles) return;
    u32 lo = 0, hi = k;
    while (lo < hi) {
        const u32 mid = lo + ((hi - lo) >> 1);
        const int32_t tile = (int32_t)(sorted[mid] >> 32);
        if (tile < t) lo = mid + 1; else hi = mid;
    }
    ranges[t] = (t == num_tiles) ? (int32_t)k : (int32_t)lo;
}

__global__ void export_lists_kernel(const u64* __restrict__ sorted, const u32 k, const float4* __restrict__ records,
                                    int64_t* __restrict__ keys, int32_t* __restrict__ ids) {
    const u32 i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= k) return;
    const u64 pr = sorted[i];
    const u32 id = (u32)pr;
    const float depth = __ldg(records + (size_t)id * 3 + 2).y;
    const int64_t d = (int64_t)(int32_t)__float_as_uint(depth);
    keys[i] = (int64_t)((pr >> 32) << 32) | d;
    ids[i] = (int32_t)id;
}

inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

}  // namespace

int64_t plan_workspace_bytes(int n) {
    const int64_t scan_tiles = (n + kScanThreads - 1) / kScanThreads;
    return align256(sort_workspace_bytes(n)) + align256(scan_tiles * 8) + align256(sizeof(PlanTail));
}

int launch_plan(const CamParams& cp, int n, const int32_t* tiles, u64* depth_keys, u64* depth_keys_alt, u32* offsets,
                void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s) {
    DSB_REQUIRE(k_host, "plan: k_host is null");
    *k_host = 0;
    if (n == 0) return DSB_OK;
    DSB_REQUIRE(tiles && depth_keys && depth_keys_alt && offsets && ws, "plan: null pointer");
    const int64_t need = plan_workspace_bytes(n);
    if (ws_bytes < need) {
        set_error("plan: workspace of %lld bytes is smaller than the %lld needed", (long long)ws_bytes, (long long)need);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    DSB_REQUIRE(((uintptr_t)ws & 255) == 0, "plan: workspace must be 256-byte aligned");
    unsigned char* base = reinterpret_cast<unsigned char*>(ws);
    const int64_t sort_bytes = align256(sort_workspace_bytes(n));
    const int64_t scan_tiles = (n + kScanThreads - 1) / kScanThreads;
    u64* lookback = reinterpret_cast<u64*>(base + sort_bytes);
    PlanTail* tail = reinterpret_cast<PlanTail*>(base + sort_bytes + align256(scan_tiles * 8));

    DSB_CUDA_CHECK(cudaMemsetAsync(ws, 0, (size_t)need, s));

    // (depth, id) order: sort the packed (depth bits << 32 | id) words on their depth bits; ids are already ascending.
    int in_alt = 0;
    {
        StageScope scope(kStageDepthSort, s);
        int rc = launch_sort(depth_keys, depth_keys_alt, nullptr, nullptr, n, 32, 64, ws, sort_bytes, &in_alt, s);
        if (rc != DSB_OK) return rc;
        if (in_alt) DSB_CUDA_CHECK(cudaMemcpyAsync(depth_keys, depth_keys_alt, (size_t)n * 8, cudaMemcpyDeviceToDevice, s));
    }
    {
        StageScope scope(kStageScan, s);
        scan_counts_kernel<<<(unsigned)scan_tiles, kScanThreads, 0, s>>>(depth_keys, tiles, n, cp.drop_last, offsets, lookback, tail);
        DSB_LAUNCH_CHECK();
    }

    struct { u64 total; u32 counter; int status; } host_tail;
    int sort_status = 0;
    DSB_CUDA_CHECK(cudaMemcpyAsync(&host_tail, tail, sizeof(host_tail), cudaMemcpyDeviceToHost, s));
    DSB_CUDA_CHECK(cudaMemcpyAsync(&sort_status, base + sort_status_offset(), sizeof(int), cudaMemcpyDeviceToHost, s));
    DSB_CUDA_CHECK(cudaStreamSynchronize(s));
    if (host_tail.status != 0 || sort_status != 0) {
        set_error("plan: a device-side wait expired (scan %d, sort %d)", host_tail.status, sort_status);
        return DSB_ERR_DEVICE_WAIT_EXPIRED;
    }
    if (host_tail.total >= (u64)DSB_MAX_PAIRS) {
        set_error("plan: %llu (tile, splat) pairs exceed the supported maximum of 2^30 - 1", (unsigned long long)host_tail.total);
        *k_host = (int64_t)host_tail.total;
        return DSB_ERR_TOO_MANY_PAIRS;
    }
    *k_host = (int64_t)host_tail.total;
    return DSB_OK;
}

int launch_emit(const CamParams& cp, int n, int64_t k, const float* records, const int32_t* tiles,
                const u64* depth_keys_sorted, const u32* offsets, u64* pairs, const SortPlan* plan, u32* hist,
                cudaStream_t s) {
    if (n == 0 || k == 0) return DSB_OK;
    DSB_REQUIRE(records && tiles && depth_keys_sorted && offsets && pairs, "emit: null pointer");
    DSB_REQUIRE(k < DSB_MAX_PAIRS, "emit: too many pairs");
    const float4* rec4 = reinterpret_cast<const float4*>(records);
    if (hist && plan && plan->npass <= 4)
        emit_pairs_kernel<true><<<(n + 255) / 256, 256, 0, s>>>(n, (u32)k, cp.tiles_x, cp.drop_last, rec4, tiles,
                                                               depth_keys_sorted, offsets, pairs, *plan, hist);
    else {
        DSB_REQUIRE(!hist, "emit: fused digit counting supports at most 4 passes");
        emit_pairs_kernel<false><<<(n + 255) / 256, 256, 0, s>>>(n, (u32)k, cp.tiles_x, cp.drop_last, rec4, tiles,
                                                                depth_keys_sorted, offsets, pairs, SortPlan{}, nullptr);
    }
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int launch_ranges(const u64* sorted, int64_t k, int H, int W, int32_t* ranges, cudaStream_t s) {
    DSB_REQUIRE(H > 0 && W > 0 && ranges, "ranges: bad arguments");
    DSB_REQUIRE(k == 0 || sorted, "ranges: null list");
    DSB_REQUIRE(k < ((int64_t)1 << 31), "ranges: too many items");
    const int t = ((W + kTile - 1) / kTile) * ((H + kTile - 1) / kTile);
    tile_ranges_kernel<<<(t + 1 + 255) / 256, 256, 0, s>>>(sorted, (u32)k, t, ranges);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int launch_export(const u64* sorted, int64_t k, const float* records, int64_t* keys, int32_t* ids, cudaStream_t s) {
    if (k == 0) return DSB_OK;
    DSB_REQUIRE(sorted && records && keys && ids, "export: null pointer");
    export_lists_kernel<<<(unsigned)((k + 255) / 256), 256, 0, s>>>(sorted, (u32)k, reinterpret_cast<const float4*>(records), keys, ids);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace dsb

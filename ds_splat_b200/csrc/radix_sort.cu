// Stage (c): stable least-significant-digit radix sort, "onesweep" style.
//
// Takes the place of thrust::sort_by_key in the reference (cpp/rasterizer_torch.cu:70-76).  The digits of
// the requested bit range are counted once (by a histogram kernel, or by the kernel that produced the
// items: emit_pairs_kernel already knows every tile id it writes); then each digit takes ONE kernel that
// reads and writes every item exactly once: a block ranks its 4096 items, publishes its per-digit counts,
// and learns the counts of all earlier blocks by decoupled look-back (each block polls its predecessors'
// status words instead of waiting for a separate scan kernel).  Only the live bits are sorted: callers
// pass [begin_bit, end_bit), and the bits are split evenly over the passes (13 tile bits -> 7 + 6), which
// keeps the scatter runs of the first pass long.
//
// Stability (equal digits keep their input order) is what makes the result identical to the
// reference's sort: within a warp items are ranked in memory order, warps are
// ordered by a scan, blocks by the look-back.
//
// Every poll loop is bounded (kSpinLimit): on expiry the block records DSB_ERR_DEVICE_WAIT_EXPIRED in
// the workspace status word and carries on with whatever it has, so the kernel always terminates.
#include <cstddef>
#include <mutex>

#include "common.cuh"

namespace dsb {

namespace {

#ifndef DSB_SORT_THREADS
#define DSB_SORT_THREADS 256
#endif
constexpr int kThreads = DSB_SORT_THREADS;   // 256: thread d also owns digit d in the block-level steps
constexpr int kWarps = kThreads / 32;
#ifndef DSB_SORT_ITEMS
#define DSB_SORT_ITEMS 16
#endif
#define DSB_SORT_MIN_BLOCKS_HINT 4  // resident blocks per SM the passes are built for
constexpr int kItems = DSB_SORT_ITEMS;          // items per thread of the large tile (multiple of 4)
constexpr int kTileItems = kThreads * kItems;   // 4096 items per block
// Lists that would not fill the GPU with large tiles are cut into half-size tiles: a pass over such a list
// is one wave of blocks, its duration is one block's chain of dependent steps, and half the items per
// thread shortens that chain.
constexpr int kSmallItems = kItems / 2;
static_assert(kThreads == 256, "the pass kernels are validated for 256 threads (digit owners, shared-memory budget)");
constexpr int kSmallTileItems = kThreads * kSmallItems;
constexpr int64_t kSmallListLimit = (int64_t)148 * DSB_SORT_MIN_BLOCKS_HINT * kSmallTileItems;  // one wave of small tiles
__host__ __device__ constexpr int tile_items_for(int64_t k, bool force_large) {
    return (!force_large && k <= kSmallListLimit) ? kSmallTileItems : kTileItems;
}
constexpr int kRadix = 256;
constexpr u32 kFlagAggregate = 1u << 30;        // status word holds this block's own count
constexpr u32 kFlagInclusive = 1u << 31;        // status word holds the count of this and all earlier blocks
constexpr u32 kValueMask = (1u << 30) - 1;

struct SortHeader {                  // start of the workspace, zeroed before every sort
    u32 hist[kMaxSortPasses][kRadix];
    u32 tile_counter[kMaxSortPasses];
    int status;
    int pad[7];
};

// Counts all digits of all passes in one read of the keys, into per-block shared-memory counters that are
// added to the global ones at the end.
__global__ void __launch_bounds__(kThreads)
radix_histogram_kernel(const u64* __restrict__ keys, const u32 n, const SortPlan plan, u32* __restrict__ hist,
                       const long long item_stride, const long long ws_stride_u32) {
    __shared__ u32 s_hist[kMaxSortPasses][kRadix];
    keys += blockIdx.y * item_stride;     // blockIdx.y: which of the batch's independent lists
    hist += blockIdx.y * ws_stride_u32;
    for (int k = threadIdx.x; k < plan.npass * kRadix; k += kThreads) (&s_hist[0][0])[k] = 0;
    __syncthreads();
    // Four keys per thread and trip, loaded before any of them is counted, so that four loads are in flight.
    constexpr u32 kUnroll = 4;
    const u32 chunk = kThreads * kUnroll;
    for (u32 base = blockIdx.x * chunk; base < n; base += gridDim.x * chunk) {
        u64 key[kUnroll];
#pragma unroll
        for (u32 q = 0; q < kUnroll; ++q) {
            const u32 i = base + q * kThreads + threadIdx.x;
            key[q] = i < n ? keys[i] : 0ull;
        }
#pragma unroll
        for (u32 q = 0; q < kUnroll; ++q) {
            const bool valid = base + q * kThreads + threadIdx.x < n;
            for (int p = 0; p < plan.npass; ++p) {
                // one shared-memory atomic per key and pass: lanes that share a digit are serialised by the hardware,
                // which costs less than finding them with ballots first
                const u32 d = sort_digit(key[q], plan.shift[p], plan.mask[p], plan.flip[p]);
                if (valid) atomicAdd(&s_hist[p][d], 1u);
            }
        }
    }
    __syncthreads();
    for (int k = threadIdx.x; k < plan.npass * kRadix; k += kThreads) {
        const u32 c = (&s_hist[0][0])[k];
        if (c) atomicAdd(hist + k, c);
    }
}

__device__ __forceinline__ u32 block_exclusive_scan_256(u32 v, u32* s_warp_sums, int tid) {
    // exclusive prefix of v over the 256 threads of the block; s_warp_sums has kWarps entries
    const int lane = tid & 31, warp = tid >> 5;
    u32 incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    __syncthreads();  // protects s_warp_sums across consecutive calls
    if (lane == 31) s_warp_sums[warp] = incl;
    __syncthreads();
    u32 prefix = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) prefix += (w < warp) ? s_warp_sums[w] : 0u;
    return prefix + incl - v;
}

#ifndef DSB_SORT_GROUP
#define DSB_SORT_GROUP 4  // items whose ranking steps are overlapped (divides the items per thread)
#endif
#ifndef DSB_SORT_MIN_BLOCKS
#define DSB_SORT_MIN_BLOCKS 4
#endif
// the ranking loop walks a thread's items in whole groups, for both tile sizes
static_assert(DSB_SORT_ITEMS % DSB_SORT_GROUP == 0 && (DSB_SORT_ITEMS / 2) % DSB_SORT_GROUP == 0,
              "items per thread (and half of it, for short lists) must be a multiple of the ranking group");

// Where a pass finds its digit inside the 64-bit item.  A digit never straddles more than the two 32-bit
// halves, so one funnel shift (or a plain shift of the high half) replaces 64-bit shifting.
struct DigitSpec {
    int high;   // digit lies entirely in the high word
    int sh;     // shift within the chosen word / funnel
    u32 mask, flip;
};
__device__ __forceinline__ u32 digit_of(const u64 key, const DigitSpec& ds) {
    const u32 lo = (u32)key, hi = (u32)(key >> 32);
    const u32 w = ds.high ? (hi >> ds.sh) : __funnelshift_r(lo, hi, ds.sh);
    return (w & ds.mask) ^ ds.flip;
}
// Lanes holding the same NB-bit digit as the caller; digits narrower than NB have zero upper bits, which
// cost a ballot each but change nothing.  ALL: every lane of the warp holds a valid item.
template <int NB, bool ALL>
__device__ __forceinline__ u32 peers_of(const u32 d, const bool valid) {
    u32 peers = ALL ? 0xffffffffu : __ballot_sync(0xffffffffu, valid);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const bool bit = (d >> b) & 1u;
        const u32 vote = __ballot_sync(0xffffffffu, bit);
        peers &= bit ? vote : ~vote;
    }
    return peers;
}

struct SweepShared {
    u64* keys;        // [kTileItems]
    u32* vals;        // [kTileItems] when values travel with the keys
    u32* wcnt;        // [kWarps][kRadix] per-warp digit counts, later first slot of (warp, digit)
    u32* glob;        // [kRadix] global position of slot p with digit d is glob[d] + p
    u32* wsum;        // [kWarps]
};

// One block-sized tile of one pass.  FULL: the tile holds kTileItems items, so no bounds checks.
template <bool HAS_VALS, int NB, int ITEMS, bool FULL>
__device__ __forceinline__ void sweep_tile(const u64* __restrict__ kin, u64* __restrict__ kout, const u32* __restrict__ vin,
                                           u32* __restrict__ vout, const u32 n, const DigitSpec ds,
                                           const u32* __restrict__ hist, u32* __restrict__ lookback, int* __restrict__ status,
                                           int* __restrict__ device_status, const u32 spin_limit, const u32 tile,
                                           const SweepShared sh) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const u32 tile_base = tile * (u32)(kThreads * ITEMS);
    const u32 tile_n = FULL ? (u32)(kThreads * ITEMS) : n - tile_base;
    const u32 wbase = tile_base + (u32)warp * (32 * ITEMS);
    u32* my_wcnt = sh.wcnt + warp * kRadix;

    // Load: item i of lane l sits at wbase + 32 i + l, so (i, l) order is memory order.  Only the digits are kept
    // (rd[i], later joined by the rank): the keys are read again, from L2, when they are moved -- sixteen 64-bit
    // keys held in registers across the ranking cost more in spills and occupancy than the second read.
#ifndef DSB_SORT_RELOAD
#define DSB_SORT_RELOAD 1
#endif
    constexpr bool kReload = DSB_SORT_RELOAD != 0;
    u64 key[ITEMS];
    u32 rd[ITEMS];
    const u64* src = kin + wbase + lane;
    const u32* vsrc = HAS_VALS ? vin + wbase + lane : nullptr;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const bool ok = FULL || wbase + 32 * i + lane < n;
        key[i] = ok ? src[32 * i] : ~0ull;
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) rd[i] = digit_of(key[i], ds);

    // Rank inside the warp: lanes holding the same digit find each other (peers_of); the lowest of them
    // bumps the warp's counter for that digit by the group size with a shared-memory atomic, whose old value
    // is the number of equal digits among the warp's earlier items.  Items are handled in groups: first all
    // peer masks, then the atomics in item order (a warp barrier between two of them keeps that order), and
    // only then the broadcasts of the old values -- so no item waits for the previous item's round trip.
    // rd[i] packs the item's rank among equal digits of its warp (low 16 bits) with its digit (bits 16..23).
    const u32 lanemask_lt = (1u << lane) - 1u;
    constexpr int kGroup = DSB_SORT_GROUP;
#pragma unroll
    for (int i0 = 0; i0 < ITEMS; i0 += kGroup) {
        u32 m[kGroup], d[kGroup], before[kGroup];
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const bool valid = FULL || wbase + 32 * (i0 + j) + lane < n;
            d[j] = rd[i0 + j];
            m[j] = peers_of<NB, FULL>(d[j], valid);
        }
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const bool valid = FULL || wbase + 32 * (i0 + j) + lane < n;
            before[j] = 0;
            if ((m[j] & lanemask_lt) == 0 && valid) before[j] = atomicAdd(&my_wcnt[d[j]], (u32)__popc(m[j]));
            __syncwarp();
        }
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const bool valid = FULL || wbase + 32 * (i0 + j) + lane < n;
            const u32 b = __shfl_sync(0xffffffffu, before[j], valid ? __ffs(m[j]) - 1 : lane);
            rd[i0 + j] = (b + (u32)__popc(m[j] & lanemask_lt)) | (d[j] << 16);
        }
    }
    __syncthreads();

    // Thread d (d < 256) owns digit d: add up the warps, publish the block's count, find the digit's first slot.
    const bool owner = tid < kRadix;
    u32 total = 0;
    volatile u32* my_status = lookback + (size_t)tile * kRadix + (owner ? tid : 0);
    if (owner) {
#pragma unroll
        for (int w = 0; w < kWarps; ++w) total += sh.wcnt[w * kRadix + tid];
        *my_status = total | (tile == 0 ? kFlagInclusive : kFlagAggregate);
    }

    const u32 dstart = block_exclusive_scan_256(total, sh.wsum, tid);
    const u32 gstart = block_exclusive_scan_256(owner ? hist[tid] : 0u, sh.wsum, tid);
    if (owner) {
        u32 run = dstart;   // wcnt[w][d] becomes the first slot of warp w's items with digit d
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const u32 c = sh.wcnt[w * kRadix + tid];
            sh.wcnt[w * kRadix + tid] = run;
            run += c;
        }
    }

    // Decoupled look-back over earlier tiles for this digit.  Measured alternatives, all slower: requesting the
    // status words of several predecessors at once (the extra registers spill); several threads per digit reading
    // as many predecessors per step; the whole block fetching the sixteen nearest rows per round with asynchronous
    // copies into the key staging area (12% slower on lists of several waves of blocks, 25% slower on one-wave
    // lists: a block's wait is covered by the other resident blocks, the extra barriers and re-fetched rows are not).
    u32 earlier = 0;
    if (tile > 0 && owner) {
        int p = (int)tile - 1;
        u32 polls = 0;
        while (p >= 0) {
            const u32 v = *(volatile const u32*)(lookback + (size_t)p * kRadix + tid);
            if ((v >> 30) == 0) {
                if (++polls > spin_limit) {
                    atomicExch(status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                    atomicExch(device_status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                    break;
                }
                __nanosleep(40);
                continue;
            }
            earlier += v & kValueMask;
            if (v & kFlagInclusive) break;
            --p;
        }
        *my_status = ((earlier + total) & kValueMask) | kFlagInclusive;
    }
    if (owner) sh.glob[tid] = gstart + earlier - dstart;
    __syncthreads();

    // Scatter into block-sorted order in shared memory, then stream out: consecutive slots of one
    // digit are consecutive in global memory, so the stores coalesce.
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        if (FULL || wbase + 32 * i + lane < n) {
            const u32 slot = my_wcnt[rd[i] >> 16] + (rd[i] & 0xffffu);
            sh.keys[slot] = kReload ? src[32 * i] : key[i];
            if (HAS_VALS) sh.vals[slot] = vsrc[32 * i];
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        const u32 slot = j * kThreads + tid;
        if (FULL || slot < tile_n) {
            const u64 k = sh.keys[slot];
            const u32 dst = sh.glob[digit_of(k, ds)] + slot;
            kout[dst] = k;
            if (HAS_VALS) vout[dst] = sh.vals[slot];
        }
    }
}

template <bool HAS_VALS, int NB, int ITEMS>
__global__ void __launch_bounds__(kThreads, DSB_SORT_MIN_BLOCKS)
onesweep_kernel(const u64* __restrict__ kin, u64* __restrict__ kout, const u32* __restrict__ vin, u32* __restrict__ vout,
                const u32 n, const DigitSpec ds, const u32* __restrict__ hist, u32* __restrict__ tile_counter,
                u32* __restrict__ lookback, int* __restrict__ status, const long long item_stride,
                const long long ws_stride_u32, int* __restrict__ device_status, const u32 spin_limit) {
    extern __shared__ __align__(16) unsigned char dyn[];
    // blockIdx.y: which of the batch's independent lists (each with its own workspace slice)
    kin += blockIdx.y * item_stride; kout += blockIdx.y * item_stride;
    if (HAS_VALS) { vin += blockIdx.y * item_stride; vout += blockIdx.y * item_stride; }
    hist += blockIdx.y * ws_stride_u32; tile_counter += blockIdx.y * ws_stride_u32;
    lookback += blockIdx.y * ws_stride_u32; status += blockIdx.y * ws_stride_u32;
    __shared__ u32 s_wcnt[kWarps * kRadix];
    __shared__ u32 s_glob[kRadix];
    __shared__ u32 s_wsum[kWarps];
    __shared__ u32 s_tile;
    SweepShared sh;
    sh.keys = reinterpret_cast<u64*>(dyn);
    sh.vals = reinterpret_cast<u32*>(dyn + kThreads * ITEMS * sizeof(u64));
    sh.wcnt = s_wcnt;
    sh.glob = s_glob;
    sh.wsum = s_wsum;

    const int tid = threadIdx.x;
    if (tid == 0) s_tile = atomicAdd(tile_counter, 1u);  // blocks take tiles in the order they start running
    for (int k = tid; k < kWarps * kRadix; k += kThreads) s_wcnt[k] = 0;
    __syncthreads();
    const u32 tile = s_tile;
    if (n - tile * (u32)(kThreads * ITEMS) >= (u32)(kThreads * ITEMS))
        sweep_tile<HAS_VALS, NB, ITEMS, true>(kin, kout, vin, vout, n, ds, hist, lookback, status, device_status, spin_limit,
                                              tile, sh);
    else
        sweep_tile<HAS_VALS, NB, ITEMS, false>(kin, kout, vin, vout, n, ds, hist, lookback, status, device_status, spin_limit,
                                               tile, sh);
}

template <bool HAS_VALS, int NB, int ITEMS>
int launch_sweep(const u64* src, u64* dst, const u32* vsrc, u32* vdst, u32 n, const DigitSpec& ds, const u32* hist,
                 u32* tile_counter, u32* lookback, int* status, int64_t tiles, size_t dyn, int batch, long long item_stride,
                 long long ws_stride_u32, cudaStream_t s, u32 spin_limit = kSpinLimit) {
    int* device_status = nullptr;
    {
        const int rc = device_status_address(&device_status);
        if (rc != DSB_OK) return rc;
    }
    // Keys alone fit the default 48 KB of shared memory per block; with values the block opts in to more.  The
    // attribute belongs to the current device's context, so it is set at every launch rather than cached.
    if (HAS_VALS || dyn + 10 * 1024 > 48 * 1024)
        DSB_CUDA_CHECK(cudaFuncSetAttribute(onesweep_kernel<HAS_VALS, NB, ITEMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    onesweep_kernel<HAS_VALS, NB, ITEMS><<<dim3((unsigned)tiles, (unsigned)batch), kThreads, dyn, s>>>(
        src, dst, vsrc, vdst, n, ds, hist, tile_counter, lookback, status, item_stride, ws_stride_u32, device_status, spin_limit);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace

// Tiles of a k-item list under the plan's tile size (0 = chosen from k).
static int64_t tiles_of(int64_t k, const SortPlan& plan) {
    const int t = plan.tile_items ? plan.tile_items : tile_items_for(k, false);
    return (k + t - 1) / t;
}

// Enough for any list of at most k items, whichever tile size it ends up with.
int64_t sort_workspace_bytes(int64_t k) {
    const int64_t small_k = k < kSmallListLimit ? k : kSmallListLimit;
    const int64_t tiles_small = (small_k + kSmallTileItems - 1) / kSmallTileItems;
    const int64_t tiles_large = (k + kTileItems - 1) / kTileItems;
    const int64_t tiles = tiles_small > tiles_large ? tiles_small : tiles_large;
    return (int64_t)sizeof(SortHeader) + (int64_t)kMaxSortPasses * tiles * kRadix * (int64_t)sizeof(u32);
}

int64_t sort_status_offset() { return (int64_t)offsetof(SortHeader, status); }

// Splits bits [begin_bit, end_bit) evenly over ceil(bits / 8) passes, low digits first.
SortPlan make_sort_plan(int begin_bit, int end_bit, bool signed_top) {
    SortPlan plan = {};
    const int bits = end_bit - begin_bit;
    plan.npass = (bits + 7) / 8;
    const int base = bits / plan.npass, extra = bits % plan.npass;
    int shift = begin_bit;
    for (int p = 0; p < plan.npass; ++p) {
        const int w = base + (p < extra ? 1 : 0);
        plan.shift[p] = shift;
        plan.bits[p] = w;
        plan.mask[p] = (1u << w) - 1u;
        plan.flip[p] = 0;
        shift += w;
        if (p == plan.npass - 1 && signed_top) plan.flip[p] = 1u << (w - 1);
    }
    return plan;
}

static int check_sort_args(const void* items, const void* items_alt, const void* ws, int64_t k, int begin_bit, int end_bit) {
    DSB_REQUIRE(begin_bit >= 0 && end_bit <= 64 && begin_bit < end_bit, "sort: bad bit range [%d, %d)", begin_bit, end_bit);
    if (k >= DSB_MAX_PAIRS) {
        set_error("sort: %lld items exceed the supported maximum of 2^30 - 1", (long long)k);
        return DSB_ERR_TOO_MANY_PAIRS;
    }
    if (k > 1) {
        DSB_REQUIRE(items && items_alt && ws, "sort: null pointer");
        DSB_REQUIRE(((uintptr_t)ws & 15) == 0, "sort: workspace must be 16-byte aligned");
    }
    return DSB_OK;
}

// A batch of `batch` equally long lists is sorted by the same launches (grid dimension y); list b uses the
// workspace slice that starts b * sort_batch_stride_bytes(k) into the workspace.
int64_t sort_batch_stride_bytes(int64_t k) { return (sort_workspace_bytes(k) + 255) / 256 * 256; }

// Step 1 of a sort whose digit counts come from the producer of the items: clears the workspace and hands
// back the histogram the producer has to fill (plan.npass rows of 256 counters).
int sort_begin(int64_t k, const SortPlan& plan, void* ws, int64_t ws_bytes, u32** hist_out, cudaStream_t s, int batch) {
    *hist_out = nullptr;
    if (k <= 1) return DSB_OK;
    const int64_t tiles = tiles_of(k, plan);
    const int64_t one = (int64_t)sizeof(SortHeader) + (int64_t)plan.npass * tiles * kRadix * (int64_t)sizeof(u32);
    const int64_t need = batch > 1 ? (int64_t)(batch - 1) * sort_batch_stride_bytes(k) + one : one;
    if (ws_bytes < need) {
        set_error("sort: workspace of %lld bytes is smaller than the %lld needed", (long long)ws_bytes, (long long)need);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    DSB_CUDA_CHECK(cudaMemsetAsync(ws, 0, (size_t)need, s));
    *hist_out = &reinterpret_cast<SortHeader*>(ws)->hist[0][0];
    return DSB_OK;
}

// Step 2: the onesweep passes, given a filled histogram.
int sort_passes(u64* items, u64* items_alt, u32* vals, u32* vals_alt, int64_t k, const SortPlan& plan, void* ws,
                int* in_alt, cudaStream_t s, int batch, int64_t item_stride) {
    if (in_alt) *in_alt = 0;
    if (k <= 1) return DSB_OK;
    const int64_t tiles = tiles_of(k, plan);
    const bool small = (plan.tile_items ? plan.tile_items : tile_items_for(k, false)) == kSmallTileItems;
    SortHeader* hdr = reinterpret_cast<SortHeader*>(ws);
    u32* lookback = reinterpret_cast<u32*>(hdr + 1);
    const size_t dyn = (small ? kSmallTileItems : kTileItems) * (sizeof(u64) + (vals ? sizeof(u32) : 0));
    const long long ws_stride_u32 = batch > 1 ? sort_batch_stride_bytes(k) / 4 : 0;
    u64 *src = items, *dst = items_alt;
    u32 *vsrc = vals, *vdst = vals_alt;
    for (int p = 0; p < plan.npass; ++p) {
        u32* lb = lookback + (size_t)p * tiles * kRadix;
        DigitSpec ds;
        ds.high = plan.shift[p] >= 32;
        ds.sh = plan.shift[p] & 31;
        ds.mask = plan.mask[p];
        ds.flip = plan.flip[p];
        const int nb = plan.bits[p] <= 5 ? 5 : plan.bits[p];
        int rc;
#define DSB_SWEEP(V, NB)                                                                                              \
    (small ? launch_sweep<V, NB, kSmallItems>(src, dst, vsrc, vdst, (u32)k, ds, hdr->hist[p], &hdr->tile_counter[p], lb,  \
                                              &hdr->status, tiles, dyn, batch, item_stride, ws_stride_u32, s)             \
           : launch_sweep<V, NB, kItems>(src, dst, vsrc, vdst, (u32)k, ds, hdr->hist[p], &hdr->tile_counter[p], lb,       \
                                         &hdr->status, tiles, dyn, batch, item_stride, ws_stride_u32, s))
        if (vals) rc = nb == 5 ? DSB_SWEEP(true, 5) : nb == 6 ? DSB_SWEEP(true, 6) : nb == 7 ? DSB_SWEEP(true, 7) : DSB_SWEEP(true, 8);
        else rc = nb == 5 ? DSB_SWEEP(false, 5) : nb == 6 ? DSB_SWEEP(false, 6) : nb == 7 ? DSB_SWEEP(false, 7) : DSB_SWEEP(false, 8);
#undef DSB_SWEEP
        if (rc != DSB_OK) return rc;
        u64* t = src; src = dst; dst = t;
        u32* tv = vsrc; vsrc = vdst; vdst = tv;
    }
    if (in_alt) *in_alt = plan.npass & 1;
    return DSB_OK;
}

// Sorts k items on bits [begin_bit, end_bit).  vals may be null.  *in_alt tells where the result is.
int launch_sort(u64* items, u64* items_alt, u32* vals, u32* vals_alt, int64_t k, int begin_bit, int end_bit,
                void* ws, int64_t ws_bytes, int* in_alt, cudaStream_t s, bool large_tiles_only, int batch,
                int64_t item_stride) {
    if (in_alt) *in_alt = 0;
    int rc = check_sort_args(items, items_alt, ws, k, begin_bit, end_bit);
    if (rc != DSB_OK) return rc;
    if (k <= 1) return DSB_OK;
    DSB_REQUIRE(!vals == !vals_alt, "sort: values and alternate values must both be given or both be null");
    SortPlan plan = make_sort_plan(begin_bit, end_bit, end_bit == 64 && vals != nullptr);  // signed keys in the pair interface
    if (large_tiles_only) plan.tile_items = kTileItems;
    // Half-size tiles pay only while the whole launch is one wave of blocks; a batch of lists fills the GPU several
    // times over even when each list alone would not.
    if ((int64_t)batch * k > kSmallListLimit) plan.tile_items = kTileItems;
    u32* hist = nullptr;
    DSB_REQUIRE(batch >= 1 && (batch == 1 || item_stride >= k), "sort: bad batch layout");
    rc = sort_begin(k, plan, ws, ws_bytes, &hist, s, batch);
    if (rc != DSB_OK) return rc;
    // Four keys per thread and trip.  Every block ends by adding its 256 counters per pass to the global ones, so
    // the grid is kept to about eight blocks per SM over the whole batch: more blocks would spend the time in
    // those atomics, fewer would leave loads uncovered.
    const int64_t chunks = (k + kThreads * 4 - 1) / (kThreads * 4);
    const int64_t per_list = (148 * 8 + batch - 1) / batch;
    const int hist_blocks = (int)(chunks < per_list ? chunks : per_list);
    radix_histogram_kernel<<<dim3((unsigned)hist_blocks, (unsigned)batch), kThreads, 0, s>>>(
        items, (u32)k, plan, hist, item_stride, batch > 1 ? sort_batch_stride_bytes(k) / 4 : 0);
    DSB_LAUNCH_CHECK();
    return sort_passes(items, items_alt, vals, vals_alt, k, plan, ws, in_alt, s, batch, item_stride);
}

// Test hook.  One histogram + ONE pass (so nothing ever reads the incomplete output) over a list of at least two
// tiles in which the tile counter starts at 1: tile 0 is never processed, never publishes its counts, and the
// block that took tile 1 polls tile 0's status words `spin_limit` times, gives up, records
// DSB_ERR_DEVICE_WAIT_EXPIRED in the workspace status word and in the device status word, and finishes like every
// other block.  All stores stay inside the buffers: a block's destination is the digit's global start plus the
// counts of earlier tiles it did see plus its own rank, which never exceeds the digit's true range.
int debug_expire_sort_wait(u64* items, u64* items_alt, int64_t k, int begin_bit, int end_bit, void* ws, int64_t ws_bytes,
                           u32 spin_limit, cudaStream_t s) {
    int rc = check_sort_args(items, items_alt, ws, k, begin_bit, end_bit);
    if (rc != DSB_OK) return rc;
    DSB_REQUIRE(end_bit - begin_bit <= 8, "debug_expire_sort_wait: one pass only (at most 8 bits)");
    DSB_REQUIRE(k >= 2 * (int64_t)kTileItems, "debug_expire_sort_wait: needs at least two tiles of %d items", kTileItems);
    DSB_REQUIRE(spin_limit >= 1 && spin_limit <= 100000, "debug_expire_sort_wait: spin_limit must be in 1..100000");
    SortPlan plan = make_sort_plan(begin_bit, end_bit, false);
    plan.tile_items = kTileItems;
    u32* hist = nullptr;
    rc = sort_begin(k, plan, ws, ws_bytes, &hist, s, 1);
    if (rc != DSB_OK) return rc;
    const int64_t chunks = (k + kThreads * 4 - 1) / (kThreads * 4);
    radix_histogram_kernel<<<dim3((unsigned)(chunks < 1184 ? chunks : 1184), 1), kThreads, 0, s>>>(items, (u32)k, plan, hist, 0, 0);
    DSB_LAUNCH_CHECK();
    SortHeader* hdr = reinterpret_cast<SortHeader*>(ws);
    static const u32 kOne = 1;
    DSB_CUDA_CHECK(cudaMemcpyAsync(&hdr->tile_counter[0], &kOne, sizeof(u32), cudaMemcpyHostToDevice, s));
    const int64_t tiles = tiles_of(k, plan);
    DigitSpec ds;
    ds.high = plan.shift[0] >= 32; ds.sh = plan.shift[0] & 31; ds.mask = plan.mask[0]; ds.flip = plan.flip[0];
    return launch_sweep<false, 8, kItems>(items, items_alt, nullptr, nullptr, (u32)k, ds, hdr->hist[0], &hdr->tile_counter[0],
                                          reinterpret_cast<u32*>(hdr + 1), &hdr->status, tiles - 1, (size_t)kTileItems * sizeof(u64),
                                          1, 0, 0, s, spin_limit);
}

// ---- sort without any allocation ------------------------------------------------------------------
// Some users of this library cannot obtain device memory at the moment they need a sort: a renderer that
// runs as a plug-in inside another engine's frame loop has usually handed every byte of the GPU to that
// engine's pool and has no right to ask the driver for more, and a latency-critical loop cannot afford
// cudaMalloc at all because it serialises the whole device.  For them the sort's scratch (digit
// histograms, tile counters, look-back status words) lives in the fixed device array below, which is part
// of the library image: every GPU that loads the library carries these ~4 MB until the process exits.
constexpr int64_t kStaticSortMaxItems = DSB_STATIC_SORT_MAX_ITEMS;
constexpr size_t kStaticSortScratchBytes =
    sizeof(SortHeader) + (size_t)kMaxSortPasses * (size_t)(kStaticSortMaxItems / kTileItems) * kRadix * sizeof(u32);
static __device__ __align__(256) unsigned char g_static_sort_scratch[kStaticSortScratchBytes];

constexpr int kMaxStaticDevices = 64;
static void* g_static_scratch_address[kMaxStaticDevices] = {};
static std::mutex g_static_scratch_mutex;

// On the host the array's name is only a handle, not an address a kernel could use; the real device
// address differs per GPU and is looked up once per device, with that device current.
static int static_scratch_for_current_device(void** out) {
    int dev = -1;
    DSB_CUDA_CHECK(cudaGetDevice(&dev));
    DSB_REQUIRE(dev >= 0 && dev < kMaxStaticDevices, "static sort: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_address[dev]) {
        void* p = nullptr;
        DSB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_sort_scratch));
        DSB_REQUIRE(p != nullptr, "static sort: the scratch array has no device address");
        g_static_scratch_address[dev] = p;
    }
    *out = g_static_scratch_address[dev];
    return DSB_OK;
}

}  // namespace dsb

extern "C" int dsb_sort_pairs_static(uint64_t* items, uint64_t* items_alt, int64_t k, int32_t begin_bit, int32_t end_bit,
                                     int32_t* sorted_in_alt_host, void* stream) {
    using namespace dsb;
    if (sorted_in_alt_host) *sorted_in_alt_host = 0;
    DSB_REQUIRE(k >= 0, "k must be non-negative");
    if (k > kStaticSortMaxItems) {
        set_error("dsb_sort_pairs_static: %lld items exceed the built-in scratch, which holds at most %lld; "
                  "use dsb_sort_pairs with a caller-provided workspace for larger lists",
                  (long long)k, (long long)kStaticSortMaxItems);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != DSB_OK) return rc;
    int in_alt = 0;
    // launch_sort clears the part of the scratch it is about to use, so whatever the previous call left
    // behind does not matter; it issues memset + kernels only, nothing that allocates.
    const int rc2 = launch_sort(reinterpret_cast<u64*>(items), reinterpret_cast<u64*>(items_alt), nullptr, nullptr, k,
                                begin_bit, end_bit, scratch, (int64_t)kStaticSortScratchBytes, &in_alt, (cudaStream_t)stream,
                                /*large_tiles_only=*/true);  // the scratch is sized for 4096-item tiles
    if (sorted_in_alt_host) *sorted_in_alt_host = in_alt;
    return rc2;
}

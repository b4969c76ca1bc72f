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

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;                      // consecutive items per thread: eight gathers in flight
constexpr int kScanTile = kScanThreads * kScanItems;
constexpr u64 kScanAggregate = 1ull << 62;
constexpr u64 kScanInclusive = 1ull << 63;
constexpr u64 kScanValue = (1ull << 62) - 1;

struct PlanTail {       // lives after the sort workspace
    u64 total;          // pairs of the view
    u64 total_rows;     // row items of the view (row-binned plans; 0 otherwise)
    u32 tile_counter;
    int status;
    u64 pad;
};
struct ScanViews {      // row-binned plans: every view's records (for the rectangles) and layout block (for K)
    const float4* records[DSB_MAX_BATCH_VIEWS];
    const u32* row_info[DSB_MAX_BATCH_VIEWS];
};

// Single-pass exclusive scan, in depth order, of the splats' tile counts (ROWS = false: offsets = first pair of every
// splat) or of the heights of their tile rectangles (ROWS = true: offsets = first row item of every splat).
template <bool ROWS>
__global__ void __launch_bounds__(kScanThreads)
scan_counts_kernel(const u64* __restrict__ depth_keys_sorted, const int32_t* __restrict__ tiles, const int n,
                   const int drop_last, u32* __restrict__ offsets, u64* __restrict__ lookback, PlanTail* __restrict__ tail,
                   const long long item_stride, const long long lookback_stride, int* __restrict__ device_status,
                   const u32 spin_limit, const ScanViews sv) {
    __shared__ u32 s_wsum[32];
    // blockIdx.y: which view of the batch (each with its own keys, counts, offsets, look-back row and tail)
    depth_keys_sorted += blockIdx.y * item_stride; tiles += blockIdx.y * item_stride; offsets += blockIdx.y * item_stride;
    lookback += blockIdx.y * lookback_stride; tail += blockIdx.y;
    __shared__ u32 s_tile;
    __shared__ u64 s_prefix;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tile = atomicAdd(&tail->tile_counter, 1u);
    __syncthreads();
    const u32 tile = s_tile;
    const int j0 = (int)tile * kScanTile + tid * kScanItems;
    u32 id[kScanItems], c[kScanItems];
#pragma unroll
    for (int q = 0; q < kScanItems; ++q) id[q] = j0 + q < n ? (u32)depth_keys_sorted[j0 + q] : 0u;
    u32 mine = 0;
#pragma unroll
    for (int q = 0; q < kScanItems; ++q) {
        c[q] = j0 + q < n ? (u32)tiles[id[q]] : 0u;
        if (drop_last && id[q] == (u32)(n - 1)) c[q] = 0;  // the reference never emits pairs for the last splat
        if (ROWS && c[q]) {                                // height of the tile rectangle
            const u32 ry = __float_as_uint(__ldg(sv.records[blockIdx.y] + (size_t)id[q] * 3 + 2).w);
            c[q] = (ry >> 16) - (ry & 0xffffu);
        }
        mine += c[q];
    }
    u32 incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        u32 w = lane < kScanThreads / 32 ? s_wsum[lane] : 0u;
        u32 wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += t;
        }
        s_wsum[lane] = wi - w;  // exclusive prefix of the warps
        const u64 block_total = __shfl_sync(0xffffffffu, wi, 31);
        volatile u64* mine = lookback + tile;
        if (lane == 0) *mine = block_total | (tile == 0 ? kScanInclusive : kScanAggregate);
        // Look-back by the whole warp: lane l reads the status of tile (p - l); the leading run of published
        // tiles, up to and including the first inclusive one, is summed at once.
        u64 earlier = 0;
        if (tile > 0) {
            int p = (int)tile - 1;
            u32 polls = 0;
            bool done = false;
            while (!done) {
                const int idx = p - lane;
                const u64 v = idx >= 0 ? *(volatile const u64*)(lookback + idx) : kScanInclusive;  // before tile 0: zero
                const u32 ready = __ballot_sync(0xffffffffu, (v >> 62) != 0);
                const u32 incl = __ballot_sync(0xffffffffu, (v & kScanInclusive) != 0);
                const int n_ready = ready == 0xffffffffu ? 32 : __ffs(~ready) - 1;
                const u32 incl_in = n_ready == 32 ? incl : (incl & ((1u << n_ready) - 1u));
                const int take = incl_in ? __ffs(incl_in) : n_ready;
                u64 part = lane < take ? (v & kScanValue) : 0ull;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                earlier += part;
                p -= take;
                done = incl_in != 0;
                if (!done && take < 32) {  // met a tile that has not published yet
                    if (++polls > spin_limit) {
                        if (lane == 0) {
                            atomicExch(&tail->status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                            atomicExch(device_status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                        }
                        break;
                    }
                    __nanosleep(40);
                }
            }
            if (lane == 0) *mine = ((earlier + block_total) & kScanValue) | kScanInclusive;
        }
        if (lane == 0) {
            s_prefix = earlier;
            if ((int)tile == (n + kScanTile - 1) / kScanTile - 1) {
                if (ROWS) {
                    tail->total_rows = earlier + block_total;
                    const u32* info = sv.row_info[blockIdx.y];   // written by the tile layout, earlier on this stream
                    tail->total = (u64)info[kRowInfoTotal] | ((u64)info[kRowInfoTotal + 1] << 32);
                } else {
                    tail->total = earlier + block_total;
                }
            }
        }
    }
    __syncthreads();
    u64 off = s_prefix + s_wsum[warp] + (incl - mine);
#pragma unroll
    for (int q = 0; q < kScanItems; ++q) {
        if (j0 + q < n) offsets[j0 + q] = off > 0xffffffffull ? 0xffffffffu : (u32)off;
        off += c[q];
    }
}

// One warp per 32 depth-ordered splats: their pair ranges are consecutive, so the warp walks the concatenated
// range 32 positions at a time and every lane writes one packed pair; all stores are consecutive 8-byte lanes.
// The splats that have pairs are first packed into the warp's low lanes (through shared memory).  In each round
// the packed splats whose range starts inside the round's 32 positions set the bit of that position; one
// warp-wide OR gives the round's start mask, and the owner of position q is the number of starts at or before q
// (a population count) plus the starts of earlier rounds -- no search.  The position inside the owner's rectangle
// is split into row and column with the width's reciprocal (integer division for rectangles of 2^20 tiles and more).
__global__ void __launch_bounds__(256)
emit_pairs_kernel(const int n, const u32 k, const int tiles_x, const int drop_last, const float4* __restrict__ records,
                  const int32_t* __restrict__ tiles, const u64* __restrict__ depth_keys_sorted,
                  const u32* __restrict__ offsets, u64* __restrict__ pairs) {
    __shared__ u32 s_id[8][32], s_tile[8][32], s_w[8][32], s_excl[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;  // position in depth order; warps are aligned to 32
    // A splat's pair count is the distance to the next splat's offset (the scan already left out the dropped last
    // splat), read along the depth order: no gather of the per-splat counts.
    u32 id = 0, c = 0, first_tile = 0, w = 1;
    const u32 off = j < n ? offsets[j] : k;
    u32 next = __shfl_down_sync(0xffffffffu, off, 1);
    if (lane == 31) next = j + 1 < n ? offsets[j + 1] : k;
    if (j < n) {
        id = (u32)depth_keys_sorted[j];
        c = next > off ? next - off : 0u;   // offsets never decrease; a caller's wrong k must not turn into a huge count
        if (c) {
            const float4 q2 = __ldg(records + (size_t)id * 3 + 2);
            const u32 rx = __float_as_uint(q2.z), ry = __float_as_uint(q2.w);
            const u32 x0 = rx & 0xffffu;
            w = (rx >> 16) - x0;
            first_tile = (ry & 0xffffu) * (u32)tiles_x + x0;
        }
    }
    u32 incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    const u32 total = __shfl_sync(0xffffffffu, incl, 31);
    if (total == 0) return;
    const u32 warp_base = __shfl_sync(0xffffffffu, off, 0);
    const u32 have = __ballot_sync(0xffffffffu, c != 0);
    const int packed = __popc(have);
    if (c) {
        const int slot = __popc(have & ((1u << lane) - 1u));
        s_id[warp][slot] = id; s_tile[warp][slot] = first_tile; s_w[warp][slot] = w; s_excl[warp][slot] = incl - c;
    }
    __syncwarp();
    const bool mine = lane < packed;
    const u32 cid = mine ? s_id[warp][lane] : 0u, ctile = mine ? s_tile[warp][lane] : 0u, cw = mine ? s_w[warp][lane] : 1u;
    const u32 cexcl = mine ? s_excl[warp][lane] : 0xffffffffu;
    float cinv;                                       // 1 / width, a few ulp off: see the split below
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(cinv) : "f"((float)cw));
    const u32 le_mask = 0xffffffffu >> (31 - lane);   // positions of the round at or before this lane's
    u32 started = 0;                                  // packed splats whose range starts before the round
    for (u32 base = 0; base < total; base += 32) {
        const u32 rel = cexcl - base;
        const u32 starts = __reduce_or_sync(0xffffffffu, (mine && rel < 32u) ? (1u << rel) : 0u);
        const int owner = (int)started + __popc(starts & le_mask) - 1;   // >= 0: position 0 of the first round is a start
        started += (u32)__popc(starts);
        const u32 o_excl = __shfl_sync(0xffffffffu, cexcl, owner);
        const u32 o_id = __shfl_sync(0xffffffffu, cid, owner);
        const u32 o_tile = __shfl_sync(0xffffffffu, ctile, owner);
        const u32 o_w = __shfl_sync(0xffffffffu, cw, owner);
        const float o_inv = __shfl_sync(0xffffffffu, cinv, owner);
        const u32 p = base + lane;
        if (p < total) {
            const u32 r = p - o_excl;
            // Row of position r in a rectangle o_w tiles wide.  (r + 0.5) / o_w lies at least 0.5 / o_w from the
            // next integer, the float product is off by less than r * 2^-21 / o_w: exact below 2^20 (checked
            // exhaustively for every width up to 300 and reciprocals up to 3 ulp off).
            const u32 row = r < (1u << 20) ? (u32)(((float)r + 0.5f) * o_inv) : r / o_w;
            const u32 tile = o_tile + row * (u32)tiles_x + (r - row * o_w);
            const u32 dst = warp_base + p;
            if (dst < k) pairs[dst] = ((u64)tile << 32) | o_id;
        }
    }
}

// From the corner marks to the tile layout, one block: prefix sums along x, then along y, turn the grid
// into pairs-per-tile; an exclusive scan in tile order gives the ranges (tile t owns sorted positions
// [ranges[t], ranges[t+1])), and every tile adds its count to the sort's digit counters.
// When the grid was worked on in shared memory its global copy is free afterwards and receives the tile
// order: the tile ids sorted by falling pair count (in 256 logarithmic classes), which the blend kernels use
// to start their longest lists first so that no long list is left running alone at the end of the launch.
constexpr int kLayoutThreads = 1024;
struct LayoutViews {       // one block per view
    int* marks[DSB_MAX_BATCH_VIEWS];
    u32* hist[DSB_MAX_BATCH_VIEWS];
    int32_t* ranges[DSB_MAX_BATCH_VIEWS];
};
__global__ void __launch_bounds__(kLayoutThreads)
tile_layout_kernel(const LayoutViews lv, const int copy_ints, const int tiles_x, const int tiles_y, const SortPlan plan,
                   const int use_smem, const int trailing_quirk, const int row_binned) {
    extern __shared__ int s_grid[];
    int* __restrict__ marks = lv.marks[blockIdx.x];
    u32* __restrict__ hist = lv.hist[blockIdx.x];
    int32_t* __restrict__ ranges = lv.ranges[blockIdx.x];
    __shared__ u32 s_hist[4][256];
    __shared__ u32 s_wsum[32];
    __shared__ u32 s_carry;
    __shared__ u64 s_last;   // (index of the last non-empty tile + 1) << 32 | start of its range; 0: no tile has pairs
    __shared__ u32 s_row_start[kRowInfoStarts];   // first list position of every tile row (row-binned images)
    __shared__ u64 s_total;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int stride = tiles_x + 1, rows = tiles_y + 1;
    if (tid == 0) { s_last = 0; s_total = 0; }
    for (int i = tid; i < 4 * 256; i += kLayoutThreads) (&s_hist[0][0])[i] = 0;
    // The grid is worked on in shared memory when it fits (up to about 4K images), else in place.
    int* diff = use_smem ? s_grid : marks;
    for (int i = tid; i < rows * stride; i += kLayoutThreads) {  // add up the copies
        int v = 0;
#pragma unroll
        for (int c = 0; c < kMarkCopies; ++c) v += marks[(size_t)c * copy_ints + i];
        diff[i] = v;
    }
    __syncthreads();
    // along x: one warp per row, 32 columns at a time with a running carry
    for (int y = warp; y < rows; y += kLayoutThreads / 32) {
        int carry = 0;
        for (int x = lane; x - lane < stride; x += 32) {
            int v = x < stride ? diff[y * stride + x] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            v += carry;
            if (x < stride) diff[y * stride + x] = v;
            carry = __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    // along y: one thread per column, eight rows in flight at a time
    for (int x = tid; x < stride; x += kLayoutThreads) {
        int acc = 0;
        for (int y0 = 0; y0 < rows; y0 += 8) {
            int v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = (y0 + q < rows) ? diff[(y0 + q) * stride + x] : 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                acc += v[q];
                if (y0 + q < rows) diff[(y0 + q) * stride + x] = acc;
            }
        }
    }
    __syncthreads();
    // exclusive scan of the per-tile counts in tile order: every thread owns a run of consecutive tiles
    const int num_tiles = tiles_x * tiles_y;
    const int per_thread = (num_tiles + kLayoutThreads - 1) / kLayoutThreads;
    const int t_begin = min(tid * per_thread, num_tiles), t_end = min(t_begin + per_thread, num_tiles);
    u32 mine = 0;
    for (int t = t_begin; t < t_end; ++t) {
        const int ty = t / tiles_x, tx = t - ty * tiles_x;
        const u32 c = (u32)max(diff[ty * stride + tx], 0);
        mine += c;
        if (c && hist && !row_binned) {
            const u64 key = (u64)(u32)t << 32;
            for (int q = 0; q < plan.npass && q < 4; ++q)
                atomicAdd(&s_hist[q][sort_digit(key, plan.shift[q], plan.mask[q], plan.flip[q])], c);
        }
    }
    u32 incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u32 v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        u32 w = s_wsum[lane], wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u32 v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        s_wsum[lane] = wi - w;
        if (lane == 31) s_carry = wi;  // grand total
    }
    __syncthreads();
    u32 running = s_wsum[warp] + incl - mine;
    u64 my_last = 0;
    {   // the pair total in 64 bits (32-bit positions wrap beyond 2^32 pairs): warp sums, then one atomic per warp
        u64 wsum = mine;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
        if (lane == 0 && wsum) atomicAdd(&s_total, wsum);
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int ty = t / tiles_x, tx = t - ty * tiles_x;
        ranges[t] = (int32_t)running;
        if (row_binned && tx == 0) s_row_start[ty] = running;
        const u32 c = (u32)max(diff[ty * stride + tx], 0);
        if (c) my_last = ((u64)(u32)(t + 1) << 32) | running;
        running += c;
    }
    if (tid == 0) ranges[num_tiles] = (int32_t)s_carry;
    if (trailing_quirk) {
        // The reference never marks the end of the last non-empty tile (see tile_ranges_kernel): the empty tiles after
        // it repeat its start, which hands its pairs to the final tile.  Reproduced when the lists are the reference's.
        if (my_last) atomicMax(&s_last, my_last);
        __syncthreads();
        const u64 last = s_last;
        if (last) {
            const int last_tile = (int)(last >> 32) - 1;
            for (int t = max(t_begin, last_tile + 1); t < t_end; ++t) ranges[t] = (int32_t)(u32)last;
        }
    }
    if (hist && !row_binned)
        for (int i = tid; i < plan.npass * 256 && i < 4 * 256; i += kLayoutThreads) hist[i] = (&s_hist[0][0])[i];
    if (hist && row_binned) {   // what row_scatter_kernel and the plan's scan read (layout of the block: common.cuh)
        __syncthreads();
        if (tid == 0) {
            s_row_start[tiles_y] = s_carry;
            hist[kRowInfoTotal] = (u32)s_total;
            hist[kRowInfoTotal + 1] = (u32)(s_total >> 32);
        }
        __syncthreads();
        if (warp == 0) {   // blocks of the scatter pass before each row: lane l takes rows 16 l .. 16 l + 15
            u32 b[16], sum = 0;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                const int r = lane * 16 + q;
                b[q] = r < tiles_y ? (s_row_start[r + 1] - s_row_start[r] + (u32)kRowTile - 1u) / (u32)kRowTile : 0u;
                sum += b[q];
            }
            u32 inc = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const u32 u = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += u;
            }
            u32 run = inc - sum;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                const int r = lane * 16 + q;
                if (r <= tiles_y) hist[r] = run;
                run += b[q];
            }
        }
        __syncthreads();
        for (int r = tid; r <= tiles_y; r += kLayoutThreads) hist[kRowInfoStarts + r] = s_row_start[r];
    }
    if (!use_smem) return;  // the grid lives in `marks` itself: no room for the order, callers fall back to tile order

    // ---- tile order by falling count: counting sort over 256 classes (exponent and three mantissa bits)
    __syncthreads();
    u32* s_class = &s_hist[0][0];  // [256] class sizes, then class offsets
    if (tid < 256) s_class[tid] = 0;
    __syncthreads();
    auto count_class = [](const u32 c) -> u32 {
        if (c == 0) return 255u;
        const int e = 31 - __clz(c);
        const u32 m = e >= 3 ? (c >> (e - 3)) & 7u : (c << (3 - e)) & 7u;
        return 254u - min(((u32)e << 3) | m, 254u);
    };
    for (int t = t_begin; t < t_end; ++t) {
        const int ty = t / tiles_x, tx = t - ty * tiles_x;
        atomicAdd(&s_class[count_class((u32)max(diff[ty * stride + tx], 0))], 1u);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the 256 class sizes, eight per lane
        u32 v[8], sum = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) { v[q] = s_class[lane * 8 + q]; sum += v[q]; }
        u32 inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u32 u = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += u;
        }
        u32 run = inc - sum;
#pragma unroll
        for (int q = 0; q < 8; ++q) { s_class[lane * 8 + q] = run; run += v[q]; }
    }
    __syncthreads();
    for (int t = t_begin; t < t_end; ++t) {
        const int ty = t / tiles_x, tx = t - ty * tiles_x;
        const u32 slot = atomicAdd(&s_class[count_class((u32)max(diff[ty * stride + tx], 0))], 1u);
        marks[slot] = t;
    }
}

// ranges[t] = number of sorted items whose tile id (high 32 bits, signed) is < t, t = 0..T -- with one habit of the
// reference kept on purpose: it marks a tile's END only where the NEXT item belongs to another tile
// (cpp/rasterizer_kernels.cu:313-322) and fills unmarked entries with a running maximum
// (cpp/rasterizer_torch.cu:37-39), so the end of the LAST non-empty tile is never marked; when empty tiles follow
// it, their entries (and the end of that tile) repeat its START, and its items fall to the final tile, whose end
// the host sets to K (:31-32).  trailing_quirk reproduces exactly that; without it the ranges are a clean partition.
__global__ void tile_ranges_kernel(const u64* __restrict__ sorted, const u32 k, const int num_tiles,
                                   int32_t* __restrict__ ranges, const int trailing_quirk) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t > num_tiles) return;
    int t_search = t;
    if (trailing_quirk && k > 0) {
        const int last_tile = (int32_t)(sorted[k - 1] >> 32);
        if (t > last_tile && t < num_tiles) t_search = max(last_tile, 0);
    }
    u32 lo = 0, hi = k;
    while (lo < hi) {
        const u32 mid = lo + ((hi - lo) >> 1);
        const int32_t tile = (int32_t)(sorted[mid] >> 32);
        if (tile < t_search) lo = mid + 1; else hi = mid;
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

// Workspace of a batch of `views` plans: per view a sort slice, then per view a scan look-back row, then the tails.
static int64_t plan_scan_row_bytes(int n) { return align256(((int64_t)n + kScanTile - 1) / kScanTile * 8); }
int64_t plan_workspace_bytes_views(int n, int views) {
    return (int64_t)views * (sort_batch_stride_bytes(n) + plan_scan_row_bytes(n)) + align256((int64_t)views * sizeof(PlanTail));
}
int64_t plan_workspace_bytes(int n) { return plan_workspace_bytes_views(n, 1); }

// Depth order and pair offsets of `views` views in the same launches.  tiles, depth_keys, depth_keys_alt and
// offsets hold one row of `n` entries per view, `item_stride` entries apart; k_host receives one total per view.
// k_host == nullptr: only the launches; read_plan_totals_views() fetches the totals later.
int launch_plan_views(const CamParams& cp, int views, int n, int64_t item_stride, const int32_t* tiles, u64* depth_keys,
                      u64* depth_keys_alt, u32* offsets, void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s,
                      const float* const* records, const u32* const* row_info, int64_t* k_rows_host) {
    DSB_REQUIRE(views >= 1 && views <= DSB_MAX_BATCH_VIEWS, "plan: between 1 and %d views per call", DSB_MAX_BATCH_VIEWS);
    DSB_REQUIRE(!records == !row_info, "plan: records and layout blocks go together");
    if (k_host)
        for (int v = 0; v < views; ++v) k_host[v] = 0;
    if (k_rows_host)
        for (int v = 0; v < views; ++v) k_rows_host[v] = 0;
    if (n == 0) return DSB_OK;
    DSB_REQUIRE(tiles && depth_keys && depth_keys_alt && offsets && ws, "plan: null pointer");
    DSB_REQUIRE(views == 1 || item_stride >= n, "plan: rows of the views overlap");
    const int64_t need = plan_workspace_bytes_views(n, views);
    if (ws_bytes < need) {
        set_error("plan: workspace of %lld bytes is smaller than the %lld needed", (long long)ws_bytes, (long long)need);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    DSB_REQUIRE(((uintptr_t)ws & 255) == 0, "plan: workspace must be 256-byte aligned");
    unsigned char* base = reinterpret_cast<unsigned char*>(ws);
    const int64_t sort_stride = sort_batch_stride_bytes(n), sort_bytes = (int64_t)views * sort_stride;
    const int64_t scan_row = plan_scan_row_bytes(n);
    const int64_t scan_tiles = ((int64_t)n + kScanTile - 1) / kScanTile;
    u64* lookback = reinterpret_cast<u64*>(base + sort_bytes);
    PlanTail* tail = reinterpret_cast<PlanTail*>(base + sort_bytes + (int64_t)views * scan_row);

    // everything, including the sort slices: a list of one item or none is not sorted and leaves its slice untouched
    DSB_CUDA_CHECK(cudaMemsetAsync(ws, 0, (size_t)need, s));

    // (depth, id) order: sort the packed (depth bits << 32 | id) words on their depth bits; ids are already ascending.
    int in_alt = 0;
    {
        StageScope scope(kStageDepthSort, s);
        int rc = launch_sort(depth_keys, depth_keys_alt, nullptr, nullptr, n, 32, 64, ws, sort_bytes, &in_alt, s, false, views,
                             item_stride);
        if (rc != DSB_OK) return rc;
        if (in_alt) {
            if (views == 1 || item_stride == n) {
                DSB_CUDA_CHECK(cudaMemcpyAsync(depth_keys, depth_keys_alt, (size_t)(item_stride * (views - 1) + n) * 8,
                                               cudaMemcpyDeviceToDevice, s));
            } else {
                DSB_CUDA_CHECK(cudaMemcpy2DAsync(depth_keys, (size_t)item_stride * 8, depth_keys_alt, (size_t)item_stride * 8,
                                                 (size_t)n * 8, (size_t)views, cudaMemcpyDeviceToDevice, s));
            }
        }
    }
    {
        StageScope scope(kStageScan, s);
        int* device_status = nullptr;
        const int rc = device_status_address(&device_status);
        if (rc != DSB_OK) return rc;
        ScanViews sv = {};
        if (records) {
            for (int v = 0; v < views; ++v) {
                DSB_REQUIRE(records[v] && row_info[v], "plan: null records or layout block for view %d", v);
                sv.records[v] = reinterpret_cast<const float4*>(records[v]);
                sv.row_info[v] = row_info[v];
            }
            scan_counts_kernel<true><<<dim3((unsigned)scan_tiles, (unsigned)views), kScanThreads, 0, s>>>(
                depth_keys, tiles, n, cp.drop_last, offsets, lookback, tail, views > 1 ? item_stride : 0, scan_row / 8,
                device_status, kSpinLimit, sv);
        } else {
            scan_counts_kernel<false><<<dim3((unsigned)scan_tiles, (unsigned)views), kScanThreads, 0, s>>>(
                depth_keys, tiles, n, cp.drop_last, offsets, lookback, tail, views > 1 ? item_stride : 0, scan_row / 8,
                device_status, kSpinLimit, sv);
        }
        DSB_LAUNCH_CHECK();
    }

    if (!k_host) return DSB_OK;
    return read_plan_totals_views(views, n, ws, ws_bytes, k_host, s, k_rows_host);
}

// The pair totals of a plan launched before on stream s (one host synchronisation), and the status words of its
// bounded waits.
int read_plan_totals_views(int views, int n, const void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s,
                           int64_t* k_rows_host) {
    DSB_REQUIRE(k_host, "plan: k_host is null");
    DSB_REQUIRE(views >= 1 && views <= DSB_MAX_BATCH_VIEWS, "plan: between 1 and %d views per call", DSB_MAX_BATCH_VIEWS);
    for (int v = 0; v < views; ++v) k_host[v] = 0;
    if (k_rows_host)
        for (int v = 0; v < views; ++v) k_rows_host[v] = 0;
    if (n == 0) return DSB_OK;
    DSB_REQUIRE(ws && ws_bytes >= plan_workspace_bytes_views(n, views), "plan: not the workspace the plan was launched with");
    const unsigned char* base = reinterpret_cast<const unsigned char*>(ws);
    const int64_t sort_stride = sort_batch_stride_bytes(n), sort_bytes = (int64_t)views * sort_stride;
    const PlanTail* tail = reinterpret_cast<const PlanTail*>(base + sort_bytes + (int64_t)views * plan_scan_row_bytes(n));
    struct HostTail { u64 total; u64 total_rows; u32 counter; int status; u64 pad; } host_tail[DSB_MAX_BATCH_VIEWS];
    int sort_status[DSB_MAX_BATCH_VIEWS] = {};
    static_assert(sizeof(HostTail) == sizeof(PlanTail), "host mirror of the plan tail");
    DSB_CUDA_CHECK(cudaMemcpyAsync(host_tail, tail, sizeof(HostTail) * views, cudaMemcpyDeviceToHost, s));
    DSB_CUDA_CHECK(cudaMemcpy2DAsync(sort_status, sizeof(int), base + sort_status_offset(), (size_t)sort_stride, sizeof(int),
                                     (size_t)views, cudaMemcpyDeviceToHost, s));
    // ... and the device's status word, which also carries what the tile sorts of earlier renders recorded
    int device_status = 0;
    {
        const int rc = begin_device_status_read(&device_status, s);
        if (rc != DSB_OK) return rc;
    }
    DSB_CUDA_CHECK(cudaStreamSynchronize(s));
    const int earlier = finish_device_status_read(device_status, s);   // clears the word when it was set
    for (int v = 0; v < views; ++v) {
        if (host_tail[v].status != 0 || sort_status[v] != 0) {
            set_error("plan: a device-side wait expired (view %d: scan %d, sort %d)", v, host_tail[v].status, sort_status[v]);
            return DSB_ERR_DEVICE_WAIT_EXPIRED;
        }
        k_host[v] = (int64_t)host_tail[v].total;
        if (k_rows_host) k_rows_host[v] = (int64_t)host_tail[v].total_rows;
    }
    if (earlier != DSB_OK) return earlier;   // recorded by a kernel outside this plan (a render's tile sort)
    for (int v = 0; v < views; ++v) {
        if (host_tail[v].total >= (u64)DSB_MAX_PAIRS) {
            set_error("plan: %llu (tile, splat) pairs exceed the supported maximum of 2^30 - 1",
                      (unsigned long long)host_tail[v].total);
            return DSB_ERR_TOO_MANY_PAIRS;
        }
    }
    return DSB_OK;
}

int launch_plan(const CamParams& cp, int n, const int32_t* tiles, u64* depth_keys, u64* depth_keys_alt, u32* offsets,
                void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s) {
    return launch_plan_views(cp, 1, n, n, tiles, depth_keys, depth_keys_alt, offsets, ws, ws_bytes, k_host, s);
}

// Test hook.  The scan of a single-view plan over at least two tiles in which the tile counter starts at 1: tile 0
// is never processed and never publishes, so the warp that took tile 1 polls it `spin_limit` times, gives up,
// records DSB_ERR_DEVICE_WAIT_EXPIRED in the plan's tail and in the device status word, and the kernel finishes.
// `ws` is laid out as launch_plan lays it out, so read_plan_totals_views() on it afterwards reports the expiry the
// way a real one would be reported.  depth_keys_sorted only has to hold splat ids below n in its low halves.
int debug_expire_scan_wait(const CamParams& cp, int n, const int32_t* tiles, const u64* depth_keys_sorted, u32* offsets,
                           void* ws, int64_t ws_bytes, u32 spin_limit, cudaStream_t s) {
    DSB_REQUIRE(tiles && depth_keys_sorted && offsets && ws, "debug_expire_scan_wait: null pointer");
    DSB_REQUIRE(n >= 2 * kScanTile, "debug_expire_scan_wait: needs at least two tiles of %d splats", kScanTile);
    DSB_REQUIRE(spin_limit >= 1 && spin_limit <= 100000, "debug_expire_scan_wait: spin_limit must be in 1..100000");
    const int64_t need = plan_workspace_bytes_views(n, 1);
    if (ws_bytes < need) {
        set_error("plan: workspace of %lld bytes is smaller than the %lld needed", (long long)ws_bytes, (long long)need);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    unsigned char* base = reinterpret_cast<unsigned char*>(ws);
    const int64_t sort_bytes = sort_batch_stride_bytes(n);
    const int64_t scan_tiles = ((int64_t)n + kScanTile - 1) / kScanTile;
    u64* lookback = reinterpret_cast<u64*>(base + sort_bytes);
    PlanTail* tail = reinterpret_cast<PlanTail*>(base + sort_bytes + plan_scan_row_bytes(n));
    DSB_CUDA_CHECK(cudaMemsetAsync(ws, 0, (size_t)need, s));
    static const u32 kOne = 1;
    DSB_CUDA_CHECK(cudaMemcpyAsync(&tail->tile_counter, &kOne, sizeof(u32), cudaMemcpyHostToDevice, s));
    int* device_status = nullptr;
    const int rc = device_status_address(&device_status);
    if (rc != DSB_OK) return rc;
    scan_counts_kernel<false><<<dim3((unsigned)(scan_tiles - 1), 1), kScanThreads, 0, s>>>(
        depth_keys_sorted, tiles, n, cp.drop_last, offsets, lookback, tail, 0, plan_scan_row_bytes(n) / 8, device_status,
        spin_limit, ScanViews{});
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int launch_emit(const CamParams& cp, int n, int64_t k, const float* records, const int32_t* tiles,
                const u64* depth_keys_sorted, const u32* offsets, u64* pairs, cudaStream_t s) {
    if (n == 0 || k == 0) return DSB_OK;
    DSB_REQUIRE(records && tiles && depth_keys_sorted && offsets && pairs, "emit: null pointer");
    DSB_REQUIRE(k < DSB_MAX_PAIRS, "emit: too many pairs");
    emit_pairs_kernel<<<(n + 255) / 256, 256, 0, s>>>(n, (u32)k, cp.tiles_x, cp.drop_last,
                                                     reinterpret_cast<const float4*>(records), tiles, depth_keys_sorted,
                                                     offsets, pairs);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int64_t tile_marks_copy_ints(int H, int W) {
    const int64_t tx = (W + kTile - 1) / kTile, ty = (H + kTile - 1) / kTile;
    return align256((tx + 1) * (ty + 1) * 4) / 4;
}

int64_t tile_marks_bytes(int H, int W) { return tile_marks_copy_ints(H, W) * 4 * kMarkCopies; }

// tile_marks: the grid the preprocess kernel filled (destroyed here); hist: the tile sort's digit counters
// (plan.npass rows of 256, may be null when there is nothing to sort); ranges: [tiles + 1].
bool tile_order_available(int H, int W) {
    const int tx = (W + kTile - 1) / kTile, ty = (H + kTile - 1) / kTile;
    return (size_t)(tx + 1) * (ty + 1) * sizeof(int) <= 200 * 1024;
}

// *has_order tells whether tile_marks[0 .. tiles) holds the tile order afterwards.  One block per view.
int launch_tile_layout_views(const CamParams& cp, int count, int* const* tile_marks, const SortPlan& plan, u32* const* hist,
                             int32_t* const* ranges, int* has_order, cudaStream_t s) {
    DSB_REQUIRE(count >= 1 && count <= DSB_MAX_BATCH_VIEWS, "tile_layout: between 1 and %d views", DSB_MAX_BATCH_VIEWS);
    DSB_REQUIRE(plan.npass <= 4, "tile_layout: at most 4 digit passes");
    DSB_REQUIRE(!row_binned(cp) || hist, "tile_layout: a row-binned image needs its layout block");
    LayoutViews lv;
    for (int v = 0; v < count; ++v) {
        DSB_REQUIRE(tile_marks[v] && ranges[v], "tile_layout: null pointer");
        lv.marks[v] = tile_marks[v];
        lv.hist[v] = hist ? hist[v] : nullptr;
        lv.ranges[v] = ranges[v];
    }
    const size_t grid_bytes = (size_t)(cp.tiles_x + 1) * (cp.tiles_y + 1) * sizeof(int);
    const int use_smem = tile_order_available(cp.H, cp.W);
    if (has_order) *has_order = use_smem;
    if (use_smem && grid_bytes > 40 * 1024)
        DSB_CUDA_CHECK(cudaFuncSetAttribute(tile_layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)grid_bytes));
    // lists identical to the reference's (its rectangles, its dropped last splat): keep its range habit too
    const int trailing_quirk = cp.drop_last && !cp.tight_tiles && cp.band_y0 == 0 && cp.band_y1 == cp.tiles_y;
    tile_layout_kernel<<<count, kLayoutThreads, use_smem ? grid_bytes : 0, s>>>(lv, (int)tile_marks_copy_ints(cp.H, cp.W),
                                                                               cp.tiles_x, cp.tiles_y, plan, use_smem, trailing_quirk,
                                                                               row_binned(cp) ? 1 : 0);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int launch_tile_layout(const CamParams& cp, int* tile_marks, const SortPlan& plan, u32* hist, int32_t* ranges,
                       int* has_order, cudaStream_t s) {
    return launch_tile_layout_views(cp, 1, &tile_marks, plan, hist ? &hist : nullptr, &ranges, has_order, s);
}

SortPlan tile_sort_plan(const CamParams& cp) {   // only the tile id is sorted: ceil(log2(tiles)) live bits above bit 32
    int tile_bits = 1;
    while ((1 << tile_bits) < cp.tiles_x * cp.tiles_y) ++tile_bits;
    return make_sort_plan(32, 32 + tile_bits, false);
}

int launch_ranges(const u64* sorted, int64_t k, int H, int W, int32_t* ranges, cudaStream_t s, int trailing_quirk) {
    DSB_REQUIRE(H > 0 && W > 0 && ranges, "ranges: bad arguments");
    DSB_REQUIRE(k == 0 || sorted, "ranges: null list");
    DSB_REQUIRE(k < ((int64_t)1 << 31), "ranges: too many items");
    const int t = ((W + kTile - 1) / kTile) * ((H + kTile - 1) / kTile);
    tile_ranges_kernel<<<(t + 1 + 255) / 256, 256, 0, s>>>(sorted, (u32)k, t, ranges, trailing_quirk);
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

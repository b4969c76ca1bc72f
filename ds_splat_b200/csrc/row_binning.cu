// Stage (b)-(d) of the fused render, "row binning": from depth-ordered splats to the tile-sorted pair list with ONE
// pass over the K-sized list.
//
// The reference writes one 64-bit key per (tile, splat) pair and sorts all of them on all 64 bits
// (cpp/rasterizer_torch.cu:70-113, cpp/rasterizer_kernels.cu:252-306).  The per-stage entry points of this library
// (dsb_emit_pairs, dsb_sort_pairs) already shrink that to a depth sort of the N splats plus a stable sort of the K
// pairs on their tile bits -- two radix passes over K items plus the pass that writes them.  The fused render goes
// one step further.  A splat's tile rectangle is a stack of ROWS of consecutive tiles, and the sorted list is
// ordered by (tile row, tile column, depth).  So:
//
//   1. every (splat, tile row) becomes one 8-byte ROW ITEM  row | first column | width | splat id , written in depth
//      order (emit_rows_kernel); there are K_rows = sum of rectangle heights of them, a third to a quarter of K;
//   2. the row items are sorted on the row (one stable radix pass of radix_sort.cu over K_rows items);
//   3. a scan of their widths gives each row item its first position in the final list (scan_widths_kernel);
//   4. row_scatter_kernel does what is left of the sort, in one pass over the K pairs that never reads a K-sized
//      list: a block takes 4096 consecutive positions of one tile row, expands the row items that cover them into
//      (tile, splat) pairs in registers, ranks them by tile column (digit = column, at most 256 columns), learns how
//      many pairs of each column the row's earlier blocks hold by decoupled look-back, and writes every pair
//      straight to its final position  ranges[tile] + earlier + rank .  The per-tile starts come from the corner-mark
//      grid (tile_layout_kernel), so no histogram of the pairs is needed either.
//
// K-sized traffic: 8 bytes written per pair, against 8 written + 2 x 16 moved before.  The list that comes out is bit
// for bit the one the reference's sort produces (rows ascending, columns ascending, depth bits ascending, ties by id).
//
// Every wait is bounded as in radix_sort.cu; tickets are taken in launch order, so a block only ever waits on
// blocks that are already running.
#include "common.cuh"

namespace dsb {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kItems = kRowScatterItems;             // pairs per thread
constexpr int kTilePairs = kRowTile;                 // pairs per block
static_assert(kTilePairs == kThreads * kItems, "row tile");
constexpr u32 kFlagAggregate = 1u << 30, kFlagInclusive = 1u << 31, kValueMask = (1u << 30) - 1;

__device__ __forceinline__ u64 pack_row_item(const u32 row, const u32 x0, const u32 w, const u32 id) {
    return ((u64)row << kRowItemRowShift) | ((u64)x0 << kRowItemX0Shift) | ((u64)w << kRowItemWShift) | id;
}

// ---- 1. row items ---------------------------------------------------------------------------------------------
// A thread takes kEmitPer splats in depth order (all their loads in flight together) and writes one item per tile
// row of each rectangle at row_offsets[j] .. ; the digit counts of the row sort are gathered on the way.
constexpr int kEmitPer = 4;
__global__ void __launch_bounds__(kThreads)
emit_rows_kernel(const int n, const u32 k_rows, const int drop_last, const float4* __restrict__ records,
                 const int32_t* __restrict__ tiles, const u64* __restrict__ depth_keys_sorted,
                 const u32* __restrict__ row_offsets, u64* __restrict__ items, const SortPlan plan, u32* __restrict__ hist) {
    __shared__ u32 s_hist[2][256];
    for (int i = threadIdx.x; i < 2 * 256; i += kThreads) (&s_hist[0][0])[i] = 0;
    __syncthreads();
    const int j0 = blockIdx.x * (kThreads * kEmitPer) + threadIdx.x;
    u32 id[kEmitPer], c[kEmitPer], off[kEmitPer];
    float4 q2[kEmitPer];
#pragma unroll
    for (int q = 0; q < kEmitPer; ++q) {
        const int j = j0 + q * kThreads;
        id[q] = j < n ? (u32)depth_keys_sorted[j] : 0u;
        off[q] = j < n ? row_offsets[j] : 0u;
    }
#pragma unroll
    for (int q = 0; q < kEmitPer; ++q) {
        c[q] = j0 + q * kThreads < n ? (u32)tiles[id[q]] : 0u;
        if (drop_last && id[q] == (u32)(n - 1)) c[q] = 0;
    }
#pragma unroll
    for (int q = 0; q < kEmitPer; ++q) q2[q] = c[q] ? __ldg(records + (size_t)id[q] * 3 + 2) : make_float4(0, 0, 0, 0);
#pragma unroll
    for (int q = 0; q < kEmitPer; ++q) {
        if (!c[q]) continue;
        const u32 rx = __float_as_uint(q2[q].z), ry = __float_as_uint(q2[q].w);
        const u32 x0 = rx & 0xffffu, w = (rx >> 16) - x0, y0 = ry & 0xffffu, h = (ry >> 16) - y0;
        for (u32 r = 0; r < h; ++r) {
            const u64 item = pack_row_item(y0 + r, x0, w, id[q]);
            if (off[q] + r < k_rows) items[off[q] + r] = item;
            for (int p = 0; p < plan.npass; ++p)
                atomicAdd(&s_hist[p][sort_digit(item, plan.shift[p], plan.mask[p], plan.flip[p])], 1u);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < plan.npass * 256; i += kThreads) {
        const u32 v = (&s_hist[0][0])[i];
        if (v) atomicAdd(hist + i, v);
    }
}

// ---- 3. first final-list position of every sorted row item ---------------------------------------------------
constexpr int kScanItems = 16, kScanTile = kThreads * kScanItems;   // a thread's items are consecutive: 128-byte runs
constexpr u64 kScanAggregate = 1ull << 62, kScanInclusive = 1ull << 63, kScanValue = (1ull << 62) - 1;
struct WidthScanTail { u32 tile_counter; int status; };

// It also tells every block of the scatter pass where to start: block_info[b] = the row item that covers the block's
// first position | its tile row << 32 (b = blocks before that row + chunk within the row; all ones: no such block).
__global__ void __launch_bounds__(kThreads)
scan_widths_kernel(const u64* __restrict__ items, const u32 k_rows, u32* __restrict__ first_pos, u64* __restrict__ lookback,
                   WidthScanTail* __restrict__ tail, int* __restrict__ device_status, const u32 spin_limit,
                   const u32* __restrict__ row_info, const int tiles_y, u64* __restrict__ block_info) {
    __shared__ u32 s_wsum[32];
    __shared__ u32 s_tile;
    __shared__ u64 s_prefix;
    __shared__ u32 s_row_blocks[kRowInfoStarts], s_row_start[kRowInfoStarts];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tile = atomicAdd(&tail->tile_counter, 1u);
    for (int r = tid; r <= tiles_y; r += kThreads) {
        s_row_blocks[r] = row_info[r];
        s_row_start[r] = row_info[kRowInfoStarts + r];
    }
    __syncthreads();
    const u32 tile = s_tile;
    const u32 j0 = tile * kScanTile + tid * kScanItems;
    u32 cw[kScanItems], mine = 0;   // cw: row << 16 | width
    if (j0 + kScanItems <= k_rows) {
        const ulonglong2* src = reinterpret_cast<const ulonglong2*>(items + j0);   // j0 is a multiple of 16: 16-byte aligned
#pragma unroll
        for (int q = 0; q < kScanItems; q += 2) {
            const ulonglong2 two = src[q >> 1];
            cw[q] = ((u32)(two.x >> kRowItemWShift) & kRowItemFieldMask) | ((u32)(two.x >> kRowItemRowShift) << 16);
            cw[q + 1] = ((u32)(two.y >> kRowItemWShift) & kRowItemFieldMask) | ((u32)(two.y >> kRowItemRowShift) << 16);
        }
    } else {
#pragma unroll
        for (int q = 0; q < kScanItems; ++q) {
            const u64 item = j0 + q < k_rows ? items[j0 + q] : 0ull;
            cw[q] = ((u32)(item >> kRowItemWShift) & kRowItemFieldMask) | ((u32)(item >> kRowItemRowShift) << 16);
        }
    }
#pragma unroll
    for (int q = 0; q < kScanItems; ++q) mine += cw[q] & 0xffffu;
    u32 incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        u32 w = lane < kWarps ? s_wsum[lane] : 0u, wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const u32 t = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += t;
        }
        s_wsum[lane] = wi - w;
        const u64 block_total = __shfl_sync(0xffffffffu, wi, 31);
        volatile u64* mine_word = lookback + tile;
        if (lane == 0) *mine_word = block_total | (tile == 0 ? kScanInclusive : kScanAggregate);
        u64 earlier = 0;
        if (tile > 0) {   // the whole warp looks back: lane l reads tile (p - l)
            int p = (int)tile - 1;
            u32 polls = 0;
            bool done = false;
            while (!done) {
                const int idx = p - lane;
                const u64 v = idx >= 0 ? *(volatile const u64*)(lookback + idx) : kScanInclusive;
                const u32 ready = __ballot_sync(0xffffffffu, (v >> 62) != 0);
                const u32 inc = __ballot_sync(0xffffffffu, (v & kScanInclusive) != 0);
                const int n_ready = ready == 0xffffffffu ? 32 : __ffs(~ready) - 1;
                const u32 inc_in = n_ready == 32 ? inc : (inc & ((1u << n_ready) - 1u));
                const int take = inc_in ? __ffs(inc_in) : n_ready;
                u64 part = lane < take ? (v & kScanValue) : 0ull;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                earlier += part;
                p -= take;
                done = inc_in != 0;
                if (!done && take < 32) {
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
            if (lane == 0) *mine_word = ((earlier + block_total) & kScanValue) | kScanInclusive;
        }
        if (lane == 0) s_prefix = earlier;
    }
    __syncthreads();
    u64 off = s_prefix + s_wsum[warp] + (incl - mine);
#pragma unroll
    for (int q = 0; q < kScanItems; ++q) {
        const u32 width = cw[q] & 0xffffu;
        if (j0 + q < k_rows) {
            first_pos[j0 + q] = off > 0xffffffffull ? 0xffffffffu : (u32)off;
            // Does this item cover the first position of a scatter block?  (It covers at most one: widths are <= 256.)
            const u32 r = min(cw[q] >> 16, (u32)tiles_y - 1u);
            const u32 rel = (u32)off - s_row_start[r];
            const u32 chunk = (rel + (u32)kTilePairs - 1u) / (u32)kTilePairs;
            if (chunk * (u32)kTilePairs < rel + width) block_info[s_row_blocks[r] + chunk] = (u64)(j0 + q) | ((u64)r << 32);
        }
        off += width;
    }
}

// ---- 4. the one pass over the pairs ---------------------------------------------------------------------------
__device__ __forceinline__ u32 block_exclusive_scan_256(u32 v, u32* s_warp_sums, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    u32 incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const u32 t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    __syncthreads();
    if (lane == 31) s_warp_sums[warp] = incl;
    __syncthreads();
    u32 prefix = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) prefix += (w < warp) ? s_warp_sums[w] : 0u;
    return prefix + incl - v;
}

template <int NB>
__device__ __forceinline__ u32 peers_of(const u32 d, const bool valid) {
    u32 peers = __ballot_sync(0xffffffffu, valid);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const bool bit = (d >> b) & 1u;
        const u32 vote = __ballot_sync(0xffffffffu, bit);
        peers &= bit ? vote : ~vote;
    }
    return peers;
}

struct ScatterControl { u32 ticket; int status; };
constexpr u32 kNoBlock = 0xffffffffu;
constexpr u32 kFarAway = 0xffffu;       // shared-memory code of a first position beyond the block (or of no item)
constexpr u32 kBias = 256;              // first positions are kept relative to (block start - kBias): the first item may begin earlier

template <int NB>
__global__ void __launch_bounds__(kThreads, 3)
row_scatter_kernel(const u64* __restrict__ items, const u32* __restrict__ first_pos, const u32 k_rows,
                   const int32_t* __restrict__ ranges, const u32* __restrict__ row_info, const int tiles_x, const int tiles_y,
                   u64* __restrict__ pairs, const u32 k, ScatterControl* __restrict__ ctl, u32* __restrict__ lookback,
                   int* __restrict__ device_status, const u32 spin_limit, const u64* __restrict__ block_info) {
    extern __shared__ __align__(16) unsigned char dyn[];
    u64* s_keys = reinterpret_cast<u64*>(dyn);                                           // [kTilePairs], block-sorted
    unsigned short* s_first = reinterpret_cast<unsigned short*>(dyn + kTilePairs * sizeof(u64));   // [kTilePairs + 34]
    __shared__ u32 s_wcnt[kWarps * 256];
    __shared__ u32 s_glob[256];
    __shared__ u32 s_wsum[kWarps];
    __shared__ u32 s_block;
    __shared__ u64 s_info;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        const u32 t = atomicAdd(&ctl->ticket, 1u);          // blocks take (row, chunk) in the order they start running
        s_block = t;
        s_info = block_info[t];                             // the grid is no larger than that array
    }
    for (int i = tid; i < kWarps * 256; i += kThreads) s_wcnt[i] = 0;
    __syncthreads();
    const u64 info = s_info;
    if ((u32)info == kNoBlock) return;                      // a ticket beyond the last block of the last row
    const u32 block = s_block;
    const u32 i0 = (u32)info;                               // the row item that covers the block's first position
    const int row = (int)(info >> 32);
    const u32 tile0 = (u32)row * (u32)tiles_x;
    // everything the block needs from global memory, requested together
    const u32 chunk = block - row_info[row];
    const u32 row_begin = row_info[kRowInfoStarts + row], row_end = row_info[kRowInfoStarts + row + 1];
    const u32 tile_start = tid < tiles_x ? (u32)ranges[tile0 + tid] : 0u;
    const u32 p0 = row_begin + chunk * (u32)kTilePairs;    // first final-list position of the block
    const u32 p_end = min(row_end, p0 + (u32)kTilePairs);
    const u32 have = min(k_rows - i0, (u32)kTilePairs + 1u);                     // row items that can cover this block
    for (u32 q = tid; q < (u32)kTilePairs + 34u; q += kThreads) {
        u32 code = kFarAway;
        if (q < have) code = min(first_pos[i0 + q] + kBias - p0, kFarAway);      // the first item starts at most 255 before p0
        s_first[q] = (unsigned short)code;
    }
    __syncthreads();

    // Each warp expands 32 * kItems consecutive positions, 32 at a time.  Lane c first finds where chunk c of the warp
    // starts among the block's row items (binary search in shared memory).  For every chunk the warp then holds a
    // window of 32 row items, one per lane (they cover at least 32 positions); a bit map of the positions at which an
    // item starts tells every lane which item owns its position.
    const u32 wrel = (u32)warp * (32 * kItems) + kBias;                          // warp's first position, biased like s_first
    u32 my_first = 0;
    if (lane < kItems) {
        const u32 pc = wrel + 32u * lane;
        u32 lo = 0, hi = have;                              // last index with s_first <= pc
        while (hi - lo > 1) {
            const u32 mid = (lo + hi) >> 1;
            if (s_first[mid] <= pc) lo = mid; else hi = mid;
        }
        my_first = lo;
    }
    u32 ids[kItems], rd[kItems];
    const u32 lanemask_le = 0xffffffffu >> (31 - lane);
    constexpr int kHalf = kItems / 2;
#pragma unroll
    for (int h0 = 0; h0 < kItems; h0 += kHalf) {
        u32 win_id[kHalf], win_first[kHalf], win_shift[kHalf];
#pragma unroll
        for (int i = 0; i < kHalf; ++i) {
            const u32 f = __shfl_sync(0xffffffffu, my_first, h0 + i) + lane;
            win_first[i] = s_first[min(f, (u32)kTilePairs + 33u)];
            const u64 it = i0 + f < k_rows ? items[i0 + f] : 0ull;
            win_id[i] = (u32)it;
            win_shift[i] = ((u32)(it >> kRowItemX0Shift) & kRowItemFieldMask) - win_first[i];   // first column - first position
        }
#pragma unroll
        for (int i = 0; i < kHalf; ++i) {
            // One bit per position of the chunk at which a new row item starts (bit 0: the window's first item, which
            // covers the chunk's first position); a position's owner is the item of the last start bit at or below it.
            const u32 base = wrel + 32u * (h0 + i);
            const u32 rel = win_first[i] - base;                                 // wraps for the window's first item
            const u32 bit = lane == 0 ? 1u : (rel < 32u ? 1u << rel : 0u);
            const u32 starts = __reduce_or_sync(0xffffffffu, bit);
            const int o = __popc(starts & lanemask_le) - 1;
            ids[h0 + i] = __shfl_sync(0xffffffffu, win_id[i], o);
            rd[h0 + i] = (__shfl_sync(0xffffffffu, win_shift[i], o) + base + lane) & 255u;   // tile column
        }
    }

    // Rank inside the warp (as in radix_sort.cu): lanes with the same column find each other, the lowest bumps the
    // warp's counter of that column, everyone learns how many equal columns the warp saw before.
    u32* my_wcnt = s_wcnt + warp * 256;
    const u32 lanemask_lt = (1u << lane) - 1u;
    const u32 wpos = p0 + (u32)warp * (32 * kItems) + lane;                      // this lane's first position
    constexpr int kGroup = 4;
#pragma unroll
    for (int g0 = 0; g0 < kItems; g0 += kGroup) {
        u32 m[kGroup], d[kGroup], before[kGroup];
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const bool valid = wpos + 32u * (g0 + j) < p_end;
            d[j] = rd[g0 + j];
            m[j] = peers_of<NB>(d[j], valid);
        }
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const bool valid = wpos + 32u * (g0 + j) < p_end;
            before[j] = 0;
            if ((m[j] & lanemask_lt) == 0 && valid) before[j] = atomicAdd(&my_wcnt[d[j]], (u32)__popc(m[j]));
            __syncwarp();
        }
#pragma unroll
        for (int j = 0; j < kGroup; ++j) {
            const bool valid = wpos + 32u * (g0 + j) < p_end;
            const u32 b = __shfl_sync(0xffffffffu, before[j], valid ? __ffs(m[j]) - 1 : lane);
            rd[g0 + j] = (b + (u32)__popc(m[j] & lanemask_lt)) | (d[j] << 16);
        }
    }
    __syncthreads();

    // Thread d owns column d: block total, publication, first slot per warp.
    u32 total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total += s_wcnt[w * 256 + tid];
    volatile u32* my_status = lookback + (size_t)block * 256 + tid;
    *my_status = total | (chunk == 0 ? kFlagInclusive : kFlagAggregate);
    const u32 dstart = block_exclusive_scan_256(total, s_wsum, tid);
    {
        u32 run = dstart;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const u32 c = s_wcnt[w * 256 + tid];
            s_wcnt[w * 256 + tid] = run;
            run += c;
        }
    }
    // Look-back over the earlier blocks of this ROW only (they hold the tickets just before this one).
    u32 earlier = 0;
    if (chunk > 0) {
        u32 back = 1, polls = 0;
        while (back <= chunk) {
            const u32 v = *(volatile const u32*)(lookback + (size_t)(block - back) * 256 + tid);
            if ((v >> 30) == 0) {
                if (++polls > spin_limit) {
                    atomicExch(&ctl->status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                    atomicExch(device_status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                    break;
                }
                __nanosleep(40);
                continue;
            }
            earlier += v & kValueMask;
            if (v & kFlagInclusive) break;
            ++back;
        }
        *my_status = ((earlier + total) & kValueMask) | kFlagInclusive;
    }
    s_glob[tid] = tile_start + earlier - dstart;
    __syncthreads();

    // Block-sorted order in shared memory, then out: consecutive slots of one column are consecutive in the list.
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        if (wpos + 32u * i < p_end) {
            const u32 col = rd[i] >> 16;
            s_keys[my_wcnt[col] + (rd[i] & 0xffffu)] = ((u64)(tile0 + col) << 32) | ids[i];
        }
    }
    __syncthreads();
    const u32 tile_n = p_end - p0;
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
        const u32 slot = j * kThreads + tid;
        if (slot < tile_n) {
            const u64 kk = s_keys[slot];
            const u32 dst = s_glob[((u32)(kk >> 32) - tile0) & 255u] + slot;
            if (dst < k) pairs[dst] = kk;
        }
    }
}

inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

}  // namespace

bool row_binning_supported(const CamParams& cp) {
    return cp.tiles_x <= 256 && cp.tiles_y + 1 <= kRowInfoStarts && cp.tiles_y + 1 <= kRowInfoTotal - kRowInfoStarts;
}

bool row_binned(const CamParams& cp) { return cp.row_binning && row_binning_supported(cp); }

// Workspace of a fused render over k pairs and k_rows row items:
//   [row sort: header + look-back] [width scan: look-back row + tail] [scatter: control + look-back]
//   [start of every scatter block: row item | row] [first positions: u32 x k_rows] [row items: 2 x u64 x k_rows]
struct RowWorkspace {
    unsigned char *sort_ws, *scan_lookback, *scan_tail, *scatter_ctl, *scatter_lookback, *block_info, *first_pos, *items, *items_alt;
    int64_t sort_bytes, total;
};
static RowWorkspace carve_row_workspace(void* ws, int64_t k, int64_t k_rows) {
    RowWorkspace r;
    int64_t off = 0;
    auto take = [&off](int64_t bytes) { const int64_t at = off; off += align256(bytes > 0 ? bytes : 1); return at; };
    unsigned char* base = reinterpret_cast<unsigned char*>(ws);
    r.sort_bytes = sort_workspace_bytes(k_rows);
    const int64_t a_sort = take(r.sort_bytes);
    const int64_t a_scan = take(((k_rows + kScanTile - 1) / kScanTile + 1) * 8);
    const int64_t a_tail = take(sizeof(WidthScanTail));
    const int64_t a_ctl = take(sizeof(ScatterControl));
    const int64_t max_blocks = k / kTilePairs + 1024;      // every row ends in one partial block; at most 510 rows
    const int64_t a_look = take(max_blocks * 256 * 4);
    const int64_t a_binfo = take(max_blocks * 8);
    const int64_t a_first = take(k_rows * 4);
    const int64_t a_items = take(k_rows * 8);
    const int64_t a_alt = take(k_rows * 8);
    r.sort_ws = base + a_sort; r.scan_lookback = base + a_scan; r.scan_tail = base + a_tail; r.scatter_ctl = base + a_ctl;
    r.scatter_lookback = base + a_look; r.block_info = base + a_binfo; r.first_pos = base + a_first; r.items = base + a_items; r.items_alt = base + a_alt;
    r.total = off;
    return r;
}
int64_t row_workspace_bytes(int64_t k, int64_t k_rows) { return carve_row_workspace(nullptr, k, k_rows).total; }

// From depth-ordered splats to the sorted pair list in `pairs` (see the head of this file).  row_offsets: first row
// item of every depth-ordered splat (scan of the plan); ranges / row_info: what tile_layout_kernel left.
int launch_row_binning(const CamParams& cp, int n, int64_t k, int64_t k_rows, const float* records, const int32_t* tiles,
                       const u64* depth_keys_sorted, const u32* row_offsets, const int32_t* ranges, const u32* row_info,
                       u64* pairs, void* ws, int64_t ws_bytes, cudaStream_t s) {
    if (n == 0 || k == 0 || k_rows == 0) return DSB_OK;
    DSB_REQUIRE(row_binning_supported(cp), "row binning: image of %d x %d tiles is outside its limits", cp.tiles_x, cp.tiles_y);
    DSB_REQUIRE(records && tiles && depth_keys_sorted && row_offsets && ranges && row_info && pairs && ws, "row binning: null pointer");
    DSB_REQUIRE(k < DSB_MAX_PAIRS && k_rows <= k, "row binning: bad counts (%lld pairs, %lld row items)", (long long)k, (long long)k_rows);
    DSB_REQUIRE(((uintptr_t)ws & 255) == 0, "row binning: workspace must be 256-byte aligned");
    const RowWorkspace w = carve_row_workspace(ws, k, k_rows);
    if (ws_bytes < w.total) {
        set_error("render: workspace of %lld bytes is smaller than the %lld needed", (long long)ws_bytes, (long long)w.total);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    int* device_status = nullptr;
    int rc = device_status_address(&device_status);
    if (rc != DSB_OK) return rc;
    int row_bits = 1;
    while ((1 << row_bits) < cp.tiles_y) ++row_bits;
    const SortPlan plan = make_sort_plan(kRowItemRowShift, kRowItemRowShift + row_bits, false);
    DSB_REQUIRE(plan.npass <= 2, "row binning: too many tile rows");
    u64* items = reinterpret_cast<u64*>(w.items);
    u64* items_alt = reinterpret_cast<u64*>(w.items_alt);
    {
        StageScope scope(kStageEmit, s);
        u32* hist = nullptr;
        rc = sort_begin(k_rows, plan, w.sort_ws, w.sort_bytes, &hist, s);
        if (rc != DSB_OK) return rc;
        // scan tail, scatter control and the scatter's look-back words start from zero
        DSB_CUDA_CHECK(cudaMemsetAsync(w.scan_lookback, 0, (size_t)(w.block_info - w.scan_lookback), s));
        DSB_CUDA_CHECK(cudaMemsetAsync(w.block_info, 0xff, (size_t)(w.first_pos - w.block_info), s));   // "no such block"
        if (k_rows > 1) {
            emit_rows_kernel<<<(n + kThreads * kEmitPer - 1) / (kThreads * kEmitPer), kThreads, 0, s>>>(
                n, (u32)k_rows, cp.drop_last, reinterpret_cast<const float4*>(records), tiles, depth_keys_sorted, row_offsets,
                items, plan, hist);
        } else {   // a single row item is not sorted and has no histogram to fill
            SortPlan none = plan; none.npass = 0;
            emit_rows_kernel<<<(n + kThreads * kEmitPer - 1) / (kThreads * kEmitPer), kThreads, 0, s>>>(
                n, (u32)k_rows, cp.drop_last, reinterpret_cast<const float4*>(records), tiles, depth_keys_sorted, row_offsets,
                items, none, nullptr);
        }
        DSB_LAUNCH_CHECK();
    }
    StageScope scope(kStageTileSort, s);
    int in_alt = 0;
    rc = sort_passes(items, items_alt, nullptr, nullptr, k_rows, plan, w.sort_ws, &in_alt, s);
    if (rc != DSB_OK) return rc;
    const u64* sorted_items = in_alt ? items_alt : items;
    u32* first_pos = reinterpret_cast<u32*>(w.first_pos);
    scan_widths_kernel<<<(unsigned)((k_rows + kScanTile - 1) / kScanTile), kThreads, 0, s>>>(
        sorted_items, (u32)k_rows, first_pos, reinterpret_cast<u64*>(w.scan_lookback),
        reinterpret_cast<WidthScanTail*>(w.scan_tail), device_status, kSpinLimit, row_info, cp.tiles_y,
        reinterpret_cast<u64*>(w.block_info));
    DSB_LAUNCH_CHECK();
    const int64_t max_blocks = k / kTilePairs + cp.tiles_y;
    const size_t dyn = (size_t)kTilePairs * sizeof(u64) + ((size_t)kTilePairs + 34) * sizeof(unsigned short);
    auto launch = [&](auto kernel) -> int {
        // static + dynamic shared memory pass the 48 KB a block gets without asking; the attribute belongs to the
        // current device's context, so it is set at every launch rather than cached
        DSB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
        kernel<<<(unsigned)max_blocks, kThreads, dyn, s>>>(sorted_items, first_pos, (u32)k_rows, ranges, row_info, cp.tiles_x,
                                                          cp.tiles_y, pairs, (u32)k, reinterpret_cast<ScatterControl*>(w.scatter_ctl),
                                                          reinterpret_cast<u32*>(w.scatter_lookback), device_status, kSpinLimit,
                                                          reinterpret_cast<const u64*>(w.block_info));
        DSB_LAUNCH_CHECK();
        return DSB_OK;
    };
    int col_bits = 1;
    while ((1 << col_bits) < cp.tiles_x) ++col_bits;
    if (col_bits <= 5) return launch(row_scatter_kernel<5>);
    if (col_bits == 6) return launch(row_scatter_kernel<6>);
    if (col_bits == 7) return launch(row_scatter_kernel<7>);
    return launch(row_scatter_kernel<8>);
}

}  // namespace dsb

// Row permutation that groups output rows with equal kernel-offset masks, so that
// the 256-row tiles of the tensor-core convolution see few distinct offsets each
// (the idea of the reference's mask-sorted view, core/relations/views.py:467-510,
// built natively). Stable LSD radix sort of (mask, row) with 10-bit digits. A pass is
// three launches over 4096-row tiles (8 warps x 512 rows): per-tile digit histograms,
// a column scan over the tiles, and a scatter that ranks equal digits inside a tile in
// row order (warp match/ballot inside a 32-row step, running per-warp counters across
// steps, a prefix over the warps) -- no atomics, so the permutation is a pure function
// of the masks. The first pass reads the masks directly (rows at or beyond counts[1]
// get a key above every mask and therefore sort last), the last one writes only the
// permutation. Only the digits that can differ are sorted: ceil((K + 1) / 10) passes
// (three for a 3x3x3 kernel, one for a 2x2x2 one).
#include <algorithm>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kDigitBits = 10;
constexpr int kBuckets = 1 << kDigitBits;
constexpr int kBinsPerThread = kBuckets / 256;
constexpr int kWarps = 8;
constexpr int kSteps = 16;                        // 32-row steps per warp
constexpr int kRowsPerWarp = 32 * kSteps;
constexpr int kTile = kWarps * kRowsPerWarp;      // 4096 rows

struct OrderKeys {
    const uint32_t* keys;      // keys of the previous pass, or
    const int32_t* row_masks;  // the masks themselves (first pass)
    const int32_t* counts;
    uint32_t inactive_key;
    int rows;

    // sort key of position i (i < rows)
    __device__ __forceinline__ uint32_t load(int i, int n_out) const {
        if (keys != nullptr) {
            return keys[i];
        }
        return i < n_out ? static_cast<uint32_t>(row_masks[i]) : inactive_key;
    }
};

// digits of this warp's 512 rows, -1 - lane beyond the end (never equal to a real digit
// or to another lane's filler)
__device__ __forceinline__ void load_digits(
    const OrderKeys& in, int first, int shift, int lane, uint32_t (&key)[kSteps], int (&digit)[kSteps]
) {
    const int n_out = in.keys != nullptr ? 0 : clamp_count(in.counts + 1, in.rows);
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
        const int i = first + s * 32 + lane;
        const bool valid = i < in.rows;
        key[s] = valid ? in.load(i, n_out) : 0u;
        digit[s] = valid ? static_cast<int>((key[s] >> shift) & (kBuckets - 1)) : -1 - lane;
    }
}

__global__ void __launch_bounds__(kWarps * 32) order_hist_kernel(
    OrderKeys in, int shift, int32_t* tile_hist
) {
    __shared__ int counts[kWarps][kBuckets];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    for (int b = lane; b < kBuckets; b += 32) {
        counts[warp][b] = 0;
    }
    __syncwarp();
    uint32_t key[kSteps];
    int digit[kSteps];
    load_digits(in, blockIdx.x * kTile + warp * kRowsPerWarp, shift, lane, key, digit);
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
        const unsigned peers = __match_any_sync(0xffffffffu, digit[s]);
        if (digit[s] >= 0 && (peers & lanemask_lt()) == 0) {
            counts[warp][digit[s]] += __popc(peers);  // one lane per distinct digit
        }
        __syncwarp();
    }
    __syncthreads();
    for (int b = threadIdx.x; b < kBuckets; b += kWarps * 32) {
        int total = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            total += counts[w][b];
        }
        tile_hist[static_cast<size_t>(blockIdx.x) * kBuckets + b] = total;
    }
}

// block b scans column b of tile_hist over the tiles (exclusive, in place)
__global__ void __launch_bounds__(256) order_scan_kernel(
    int32_t* tile_hist, int tiles, int32_t* totals
) {
    __shared__ int warp_totals[8];
    __shared__ int carry_shared;
    int column = blockIdx.x;
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        carry_shared = 0;
    }
    __syncthreads();
    for (int base = 0; base < tiles; base += 256) {
        int i = base + threadIdx.x;
        int v = i < tiles ? tile_hist[static_cast<size_t>(i) * kBuckets + column] : 0;
        int wtotal;
        int prefix = warp_exclusive_scan(v, wtotal);
        if (lane == 31) {
            warp_totals[warp] = wtotal;
        }
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) {
            before += warp_totals[w];
        }
        int carry = carry_shared;
        if (i < tiles) {
            tile_hist[static_cast<size_t>(i) * kBuckets + column] = carry + before + prefix;
        }
        __syncthreads();
        if (threadIdx.x == 255) {
            carry_shared = carry + before + prefix + v;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        totals[column] = carry_shared;
    }
}

__global__ void __launch_bounds__(kWarps * 32) order_scatter_kernel(
    OrderKeys in, const int32_t* perm_in, int shift, const int32_t* tile_hist,
    const int32_t* totals, uint32_t* keys_out, int32_t* perm_out
) {
    __shared__ int cursor[kWarps][kBuckets];
    __shared__ int warp_sums[kWarps];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    for (int b = lane; b < kBuckets; b += 32) {
        cursor[warp][b] = 0;
    }
    __syncwarp();
    const int first = blockIdx.x * kTile + warp * kRowsPerWarp;
    uint32_t key[kSteps];
    int digit[kSteps];
    int rank[kSteps];  // rank among this warp's rows with the same digit
    load_digits(in, first, shift, lane, key, digit);
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
        const unsigned peers = __match_any_sync(0xffffffffu, digit[s]);
        const int before = __popc(peers & lanemask_lt());
        rank[s] = (digit[s] >= 0 ? cursor[warp][digit[s]] : 0) + before;
        __syncwarp();
        if (digit[s] >= 0 && before == 0) {
            cursor[warp][digit[s]] += __popc(peers);
        }
        __syncwarp();
    }
    // where digit b of this tile starts: digits below b anywhere, digit b in earlier tiles.
    // Thread t owns bins kBinsPerThread * t ..: a prefix inside the thread, then over the block.
    int bin_total[kBinsPerThread];
    int thread_total = 0;
#pragma unroll
    for (int u = 0; u < kBinsPerThread; ++u) {
        bin_total[u] = __ldg(totals + threadIdx.x * kBinsPerThread + u);
        thread_total += bin_total[u];
    }
    int wtotal;
    const int below_in_warp = warp_exclusive_scan(thread_total, wtotal);
    if (lane == 31) {
        warp_sums[warp] = wtotal;
    }
    __syncthreads();
    int below = below_in_warp;
    for (int w = 0; w < warp; ++w) {
        below += warp_sums[w];
    }
#pragma unroll
    for (int u = 0; u < kBinsPerThread; ++u) {
        const int b = threadIdx.x * kBinsPerThread + u;
        int start = below + __ldg(tile_hist + static_cast<size_t>(blockIdx.x) * kBuckets + b);
        below += bin_total[u];
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const int count = cursor[w][b];
            cursor[w][b] = start;  // now: where warp w's rows with digit b start
            start += count;
        }
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
        if (digit[s] >= 0) {
            const int i = first + s * 32 + lane;
            const int pos = cursor[warp][digit[s]] + rank[s];
            if (keys_out != nullptr) {
                keys_out[pos] = key[s];
            }
            perm_out[pos] = perm_in != nullptr ? perm_in[i] : i;
        }
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

size_t lat_mask_order_workspace_bytes(int32_t rows) {
    size_t r = static_cast<size_t>(std::max(rows, 1));
    size_t tiles = (r + kTile - 1) / kTile;
    return 4 * align_up(sizeof(int32_t) * r) + align_up(sizeof(int32_t) * tiles * kBuckets) +
           align_up(sizeof(int32_t) * kBuckets) + 1024;
}

int lat_build_mask_row_order(
    const int32_t* row_masks, int32_t rows, int32_t kernel_count, const int32_t* counts,
    int32_t* row_order,
    void* workspace, size_t workspace_bytes, int32_t* status, void* stream_ptr
) {
    (void)status;
    LAT_REQUIRE(rows >= 0, "row_masks must have shape (Nout, 1).");
    LAT_REQUIRE(counts != nullptr, "counts must have shape (2,) and int32 dtype.");
    if (rows == 0) {
        return LAT_OK;
    }
    LAT_REQUIRE(row_masks != nullptr && row_order != nullptr, "row_masks and row_order are required.");
    cudaStream_t stream = as_stream(stream_ptr);
    Workspace ws(workspace, workspace_bytes);
    uint32_t* keys_a = ws.take<uint32_t>(rows);
    uint32_t* keys_b = ws.take<uint32_t>(rows);
    int32_t* perm_a = ws.take<int32_t>(rows);
    int32_t* perm_b = ws.take<int32_t>(rows);
    const int tiles = (rows + kTile - 1) / kTile;
    int32_t* hist = ws.take<int32_t>(static_cast<size_t>(tiles) * kBuckets);
    int32_t* totals = ws.take<int32_t>(kBuckets);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the row order.");
    }
    LAT_REQUIRE(kernel_count >= 1 && kernel_count <= 32, "row masks need 1 <= K <= 32.");
    // masks use bits [0, K); inactive rows get bit K (or all ones when K == 32)
    const uint32_t inactive_key = kernel_count >= 32 ? 0xFFFFFFFFu : (1u << kernel_count);
    const int passes = kernel_count >= 32 ? 4 : (kernel_count + 1 + kDigitBits - 1) / kDigitBits;
    for (int pass = 0; pass < passes; ++pass) {
        const bool last = pass == passes - 1;
        OrderKeys in{};
        in.keys = pass == 0 ? nullptr : ((pass & 1) ? keys_b : keys_a);
        in.row_masks = row_masks;
        in.counts = counts;
        in.inactive_key = inactive_key;
        in.rows = rows;
        const int32_t* pin = pass == 0 ? nullptr : ((pass & 1) ? perm_b : perm_a);
        uint32_t* kout = last ? nullptr : ((pass & 1) ? keys_a : keys_b);
        int32_t* pout = last ? row_order : ((pass & 1) ? perm_a : perm_b);
        order_hist_kernel<<<tiles, kWarps * 32, 0, stream>>>(in, pass * kDigitBits, hist);
        LAT_LAUNCH_CHECK();
        order_scan_kernel<<<kBuckets, 256, 0, stream>>>(hist, tiles, totals);
        LAT_LAUNCH_CHECK();
        order_scatter_kernel<<<tiles, kWarps * 32, 0, stream>>>(
            in, pin, pass * kDigitBits, hist, totals, kout, pout);
        LAT_LAUNCH_CHECK();
    }
    return LAT_OK;
}

} // extern "C"

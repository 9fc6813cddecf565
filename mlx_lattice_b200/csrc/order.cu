// Row permutation that groups output rows with equal kernel-offset masks, so that
// the 128-row tiles of the tensor-core convolution see few distinct offsets each
// (the idea of the reference's mask-sorted view, core/relations/views.py:467-510,
// built natively). Stable LSD radix sort of (mask, row) with 8-bit digits: per
// 1024-row chunk histograms, per-digit column scans over the chunks, then a stable
// scatter that ranks equal digits inside a chunk with warp match/ballot -- integer
// atomics only on shared counters whose final values do not depend on ordering.
// Rows at or beyond counts[1] get a key above every mask and therefore sort last. Only
// the digits that can differ are sorted: ceil((K + 1) / 8) passes for K kernel offsets.
#include <algorithm>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kChunk = 1024;
constexpr int kBuckets = 256;
constexpr int kWarps = 8;

__global__ void order_init_kernel(
    const int32_t* row_masks, int rows, const int32_t* counts, uint32_t inactive_key,
    uint32_t* keys, int32_t* perm
) {
    int n_out = clamp_count(counts + 1, rows);
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) {
        keys[i] = i < n_out ? static_cast<uint32_t>(row_masks[i]) : inactive_key;
        perm[i] = i;
    }
}

__global__ void __launch_bounds__(kWarps * 32) order_hist_kernel(
    const uint32_t* keys, int rows, int shift, int32_t* chunk_hist
) {
    __shared__ int counts[kWarps][kBuckets];
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int chunk = blockIdx.x * kWarps + warp;
    for (int b = lane; b < kBuckets; b += 32) {
        counts[warp][b] = 0;
    }
    __syncwarp();
    int begin = chunk * kChunk;
    for (int i = begin + lane; i < begin + kChunk && i < rows; i += 32) {
        atomicAdd(&counts[warp][(keys[i] >> shift) & 255u], 1);
    }
    __syncwarp();
    if (begin < rows) {
        for (int b = lane; b < kBuckets; b += 32) {
            chunk_hist[static_cast<size_t>(chunk) * kBuckets + b] = counts[warp][b];
        }
    }
}

// block b scans column b of chunk_hist over the chunks (exclusive, in place)
__global__ void __launch_bounds__(256) order_scan_kernel(
    int32_t* chunk_hist, int chunks, int32_t* totals
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
    for (int base = 0; base < chunks; base += 256) {
        int i = base + threadIdx.x;
        int v = i < chunks ? chunk_hist[static_cast<size_t>(i) * kBuckets + column] : 0;
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
        if (i < chunks) {
            chunk_hist[static_cast<size_t>(i) * kBuckets + column] = carry + before + prefix;
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
    const uint32_t* keys_in, const int32_t* perm_in, int rows, int shift,
    const int32_t* chunk_hist, const int32_t* totals, uint32_t* keys_out, int32_t* perm_out
) {
    __shared__ int cursor[kWarps][kBuckets];
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    int chunk = blockIdx.x * kWarps + warp;
    int begin = chunk * kChunk;
    int run = 0;
    for (int base = 0; base < kBuckets; base += 32) {
        int b = base + lane;
        int v = __ldg(totals + b);
        int total;
        int pre = warp_exclusive_scan(v, total);
        cursor[warp][b] =
            run + pre + (begin < rows ? chunk_hist[static_cast<size_t>(chunk) * kBuckets + b] : 0);
        run += total;
    }
    __syncwarp();
    for (int base = begin; base < begin + kChunk && base < rows; base += 32) {
        int i = base + lane;
        bool valid = i < rows;
        uint32_t key = valid ? keys_in[i] : 0u;
        int digit = valid ? static_cast<int>((key >> shift) & 255u) : -1 - lane;
        unsigned peers = __match_any_sync(0xffffffffu, digit);
        int rank = __popc(peers & lanemask_lt());
        if (valid) {
            int pos = cursor[warp][digit] + rank;
            keys_out[pos] = key;
            perm_out[pos] = perm_in[i];
        }
        __syncwarp();
        if (valid && rank == 0) {
            cursor[warp][digit] += __popc(peers);
        }
        __syncwarp();
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

size_t lat_mask_order_workspace_bytes(int32_t rows) {
    size_t r = static_cast<size_t>(std::max(rows, 1));
    size_t chunks = (r + kChunk - 1) / kChunk + kWarps;
    return 4 * align_up(sizeof(int32_t) * r) + align_up(sizeof(int32_t) * chunks * kBuckets) +
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
    cudaStream_t stream = as_stream(stream_ptr);
    Workspace ws(workspace, workspace_bytes);
    uint32_t* keys_a = ws.take<uint32_t>(rows);
    uint32_t* keys_b = ws.take<uint32_t>(rows);
    int32_t* perm_a = ws.take<int32_t>(rows);
    int32_t* perm_b = ws.take<int32_t>(rows);
    int chunks = (rows + kChunk - 1) / kChunk;
    int blocks = (chunks + kWarps - 1) / kWarps;
    int32_t* hist = ws.take<int32_t>(static_cast<size_t>(blocks) * kWarps * kBuckets);
    int32_t* totals = ws.take<int32_t>(kBuckets);
    if (!ws.ok) {
        return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the row order.");
    }
    LAT_REQUIRE(kernel_count >= 1 && kernel_count <= 32, "row masks need 1 <= K <= 32.");
    // masks use bits [0, K); inactive rows get bit K (or all ones when K == 32)
    const uint32_t inactive_key = kernel_count >= 32 ? 0xFFFFFFFFu : (1u << kernel_count);
    const int passes = kernel_count >= 32 ? 4 : (kernel_count + 1 + 7) / 8;
    order_init_kernel<<<(rows + 255) / 256, 256, 0, stream>>>(
        row_masks, rows, counts, inactive_key, keys_a, perm_a);
    LAT_LAUNCH_CHECK();
    for (int pass = 0; pass < passes; ++pass) {
        const uint32_t* kin = (pass & 1) ? keys_b : keys_a;
        const int32_t* pin = (pass & 1) ? perm_b : perm_a;
        uint32_t* kout = (pass & 1) ? keys_a : keys_b;
        int32_t* pout = pass == passes - 1 ? row_order : ((pass & 1) ? perm_a : perm_b);
        order_hist_kernel<<<blocks, kWarps * 32, 0, stream>>>(kin, rows, pass * 8, hist);
        LAT_LAUNCH_CHECK();
        order_scan_kernel<<<kBuckets, 256, 0, stream>>>(hist, chunks, totals);
        LAT_LAUNCH_CHECK();
        order_scatter_kernel<<<blocks, kWarps * 32, 0, stream>>>(
            kin, pin, rows, pass * 8, hist, totals, kout, pout);
        LAT_LAUNCH_CHECK();
    }
    return LAT_OK;
}

} // extern "C"

// Tensor-core sparse convolution driven by a gather plan (conv_plan.cu): the same
// output-stationary implicit GEMM on tcgen05 as conv_tc.cu -- 256-row tiles, a unit =
// (kernel offset used by the tile, 32-channel slice of C_in), two units per 64-wide K
// slab, fp32 accumulators in TMEM, one deterministic store per output row -- but no role
// ever touches the relation's CSR arrays and the producers never synchronise with each
// other:
//   warps 0-7  producers. A thread owns one 16-byte chunk column (so one unit of each
//              slab) and the eight tile rows q, q+32, ..; the input rows of those eight
//              are 32 contiguous bytes of the plan's row vector, fetched one slab ahead
//              into registers. Per slab: wait for a free stage, 8 cp.async for A (zero
//              fill where the row has no neighbour), C_out/32 cp.async for the fp16 B
//              tile, then cp.async.mbarrier.arrive.noinc so that the stage's barrier
//              completes when the copies land. The stream of slabs runs across tile
//              boundaries; tile headers are prefetched a tile ahead. When C_in is a
//              multiple of 64 both units of a slab share their kernel offset: the loop
//              nest is tile > offset > slab with the row addresses computed once per
//              offset, and the weight tile of a slab is one TMA box
//              (cp.async.bulk.tensor.3d, 128-byte swizzle) issued by one thread.
//   warp 16    one thread issues the MMAs (8 per slab), commits the stage back to the
//              producers and, per tile, the accumulator to the epilogue.
//   warps 8-15 epilogue: tcgen05.ld, optional bias, one cast to fp16, 16-byte stores.
// Every mbarrier wait is bounded by a clock budget; on expiry the kernel records
// LAT_STATUS_WAIT_TIMEOUT, every role leaves its loop and the CTA frees its TMEM.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "conv_plan.cuh"
#include "tcgen05.cuh"

namespace lat {

using namespace tcgen05;

namespace {

constexpr int kTileRows = kPlanTileRows;
constexpr int kProducerThreads = 256;
constexpr int kEpilogueThreads = 256;
constexpr int kThreads = 544;
constexpr int kMmaWarp = 16;
constexpr int kMaxStages = 8;
constexpr int kMaxAccStages = 8;
constexpr int kSlabBytesA = kTileRows * 128;

struct PlanConvParams {
    const __half* feats;
    int feat_row_bytes;
    int c_in;
    int c_out;
    // fp16 weights addressed (in bytes) as base + k*w_k_bytes + co*w_co_bytes + 2*ci
    const __half* weights;
    long long w_k_bytes;
    long long w_co_bytes;
    const int2* tile_info;     // [num_tiles + 1]; the last entry holds (active tiles, vectors)
    const int32_t* vectors;
    const int32_t* row_order;
    int out_capacity;
    const __half* bias;
    __half* out;
    int32_t* status;
    int stages;
    int stage_bytes;     // 32 KB of A rows + the B tile
    int tmem_cols;
    int acc_cols;
    int acc_stages;
    int num_tiles;
    int b_tma;           // 1: the B tile of a slab is one TMA box (C_in a multiple of 64)
    int b_k_outer;       // tensor-map dimension order: 1 = (C_in, C_out, K), 0 = (C_in, K, C_out)
};

struct Ring {
    int index;
    uint32_t phase;
    __device__ __forceinline__ void advance(int size) {
        if (++index == size) {
            index = 0;
            phase ^= 1u;
        }
    }
};

struct Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[kMaxAccStages];
    uint64_t acc_empty[kMaxAccStages];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ int2 load_info(const PlanConvParams& p, int tile, int active) {
    return tile < active ? __ldg(p.tile_info + tile) : make_int2(0, 0);
}

// Rows of a tile none of whose rows has an edge: zeros plus bias. Warp `w` (0-7) of a role
// writes tile rows 32 w .. 32 w + 31 as one run of 16-byte pieces, lane after lane (the
// inactive tail of a static-capacity map is a contiguous stretch of rows).
__device__ __forceinline__ void fill_edgeless_rows(const PlanConvParams& p, int tile, int w, int lane) {
    const int position = tile * kTileRows + w * 32 + lane;
    int row = -1;
    if (position < p.out_capacity) {
        row = p.row_order != nullptr ? __ldg(p.row_order + position) : position;
        if (row < 0 || row >= p.out_capacity) {
            raise_status(p.status, LAT_STATUS_BAD_INDEX);
            row = -1;
        }
    }
    const int chunks = p.c_out >> 3;
    for (int idx = lane; idx < 32 * chunks; idx += 32) {
        const int r = idx / chunks;
        const int c = idx - r * chunks;
        const int target = __shfl_sync(0xffffffffu, row, r);
        uint4 piece = make_uint4(0u, 0u, 0u, 0u);
        if (p.bias != nullptr) {
            __half2 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                h[j] = __halves2half2(__ldg(p.bias + c * 8 + 2 * j), __ldg(p.bias + c * 8 + 2 * j + 1));
            }
            piece = *reinterpret_cast<uint4*>(h);
        }
        if (target >= 0) {
            reinterpret_cast<uint4*>(p.out + static_cast<size_t>(target) * p.c_out)[c] = piece;
        }
    }
}

// the tiles past the last one with an edge are shared between the producer warps (which
// run out of work first) and the epilogue warps: even and odd rounds of the tile loop
__device__ __forceinline__ bool producers_fill(int tile, int grid) { return ((tile / grid) & 1) == 0; }

__global__ void __launch_bounds__(kThreads, 1)
tc_conv_plan_kernel(PlanConvParams p, const __grid_constant__ CUtensorMap b_map) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    Control& ctl = *reinterpret_cast<Control*>(smem + p.stages * p.stage_bytes);
    volatile int* abort_flag = &ctl.abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int upo = p.c_in / 32;  // units per kernel offset
    const int grid = gridDim.x;

    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl.full[s], kProducerThreads + (p.b_tma ? 1 : 0));
            mbar_init(&ctl.empty[s], 1);
        }
        for (int a = 0; a < kMaxAccStages; ++a) {
            mbar_init(&ctl.acc_full[a], 1);
            mbar_init(&ctl.acc_empty[a], kEpilogueThreads);
        }
        ctl.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&ctl.tmem_base)),
                     "r"(static_cast<uint32_t>(p.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl.tmem_base;
    // tiles at and beyond `active` use no kernel offset at all
    const int active = min(max(__ldg(&p.tile_info[p.num_tiles].x), 0), p.num_tiles);

    if (warp < 8) {
        // ======================= producers =======================
        const int a_chunk = tid & 7;
        const int a_half = a_chunk >> 2;        // which unit of a slab this thread feeds
        const int q = tid >> 3;                 // rows q + 32 j
        const int col8 = (a_chunk & 3) * 8;
        // shared-memory offset of (row q, this chunk); rows q + 32 j are 4096 j bytes on,
        // with the same swizzle term because (q + 32 j) % 8 == q % 8. The B tile uses the
        // same offsets for output channels q + 32 i.
        const uint32_t dst0 = static_cast<uint32_t>(q * 128 + ((a_chunk ^ (q & 7)) << 4));
        const char* const feat_bytes = reinterpret_cast<const char*>(p.feats);
        const char* const weight_bytes = reinterpret_cast<const char*>(p.weights);
        const int feat_row_bytes = p.feat_row_bytes;
        const long long w_co0 = static_cast<long long>(q) * p.w_co_bytes;
        const long long w_co_step = 32LL * p.w_co_bytes;
        const int b_copies = p.c_out >> 5;  // C_out is a multiple of 32 here, or 16 (see below)
        Ring ring{0, 0u};
        bool ok = true;

        if ((upo & 1) == 0) {
            // ---- C_in a multiple of 64: both units of a slab belong to one kernel offset ----
            // The loop nest is tile > offset > slab; everything that depends on the input
            // rows (eight source addresses and their zero-fill flags) is computed once per
            // offset, and the next offset's row vector is loaded while the current one's
            // slabs are issued, so a slab costs its copies and little else.
            const int reps = upo >> 1;  // slabs per offset
            const int unit_bytes = a_half * 64 + col8 * 2;  // this thread's 16 bytes inside a 128-byte K slab
            int tile = blockIdx.x;
            int2 info = load_info(p, tile, active);
            int4 v0 = make_int4(-1, -1, -1, -1), v1 = v0;
            auto load_vector = [&](int vector_index, int4& d0, int4& d1) {
                const int4* src = reinterpret_cast<const int4*>(
                    p.vectors + static_cast<size_t>(vector_index) * kTileRows + q * 8);
                d0 = __ldg(src);
                d1 = __ldg(src + 1);
            };
            if (tile < active && info.x != 0) {
                load_vector(info.y, v0, v1);
            }
            while (tile < active && ok) {
                int next_tile = tile + grid;
                int2 next_info = load_info(p, next_tile, active);
                uint32_t rem = static_cast<uint32_t>(info.x);
                const int present = __popc(rem);
                for (int o = 0; o < present && ok; ++o) {
                    const int k = __ffs(rem) - 1;
                    rem &= rem - 1;
                    const int idx[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    const char* src[8];
                    uint32_t valid = 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        src[j] = feat_bytes + unit_bytes +
                                 static_cast<long long>(max(idx[j], 0)) * feat_row_bytes;
                        valid |= idx[j] >= 0 ? (1u << j) : 0u;
                    }
                    // the row vector of the next offset (of this tile, or the first of the
                    // next tile that has any) travels while this offset's slabs are issued
                    if (o + 1 < present) {
                        load_vector(info.y + o + 1, v0, v1);
                    } else {
                        while (next_tile < active && next_info.x == 0) {
                            next_tile += grid;
                            next_info = load_info(p, next_tile, active);
                        }
                        if (next_tile < active) {
                            load_vector(next_info.y, v0, v1);
                        }
                    }
                    for (int r = 0; r < reps; ++r) {
                        if (!mbar_wait(&ctl.empty[ring.index], ring.phase ^ 1u, abort_flag, p.status)) {
                            ok = false;
                            break;
                        }
                        const uint32_t a_addr = smem_u32(smem + ring.index * p.stage_bytes) + dst0;
                        const uint32_t b_addr = a_addr + kSlabBytesA;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            cp_async_16(a_addr + 4096 * j, src[j] + r * 128, (valid >> j) & 1u);
                        }
                        if (p.b_tma) {
                            if (tid == 0) {
                                mbar_arrive_expect_tx(&ctl.full[ring.index],
                                                      static_cast<uint32_t>(p.c_out) * 128u);
                                tma_load_3d(b_addr - dst0, &b_map, r * 64, p.b_k_outer ? 0 : k,
                                            p.b_k_outer ? k : 0, &ctl.full[ring.index]);
                            }
                        } else {
                            const char* w_src = weight_bytes + static_cast<long long>(k) * p.w_k_bytes +
                                                r * 128 + unit_bytes + w_co0;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                if (i < b_copies) {
                                    cp_async_16(b_addr + 4096 * i, w_src, true);
                                    w_src += w_co_step;
                                }
                            }
                            if ((p.c_out & 16) && q < 16) {
                                cp_async_16(b_addr + 4096 * b_copies, w_src, true);
                            }
                        }
                        cp_async_arrive_noinc(&ctl.full[ring.index]);
                        ring.advance(p.stages);
                    }
                }
                tile = next_tile;
                info = next_info;
            }
            cp_async_wait<0>();
        } else {
        // ---- general case: a slab may straddle two kernel offsets ----
        int tile = blockIdx.x;
        int2 info = load_info(p, tile, active);
        int2 next_info = load_info(p, tile + grid, active);
        int units = 0, s = 0, o = 0, slice = 0;
        uint32_t rem = 0;
        auto skip_empty_tiles = [&]() {
            while (tile < active && info.x == 0) {
                tile += grid;
                info = next_info;
                next_info = load_info(p, tile + grid, active);
            }
        };
        auto enter_tile = [&]() {
            units = __popc(static_cast<uint32_t>(info.x)) * upo;
            s = 0;
            o = 0;
            slice = a_half;
            rem = static_cast<uint32_t>(info.x);
            while (slice >= upo) {
                slice -= upo;
                ++o;
                rem &= rem - 1;
            }
        };
        int4 i0 = make_int4(-1, -1, -1, -1), i1 = i0;
        auto load_vector = [&](int4& v0, int4& v1) {
            const int4* src = reinterpret_cast<const int4*>(
                p.vectors + (static_cast<size_t>(info.y) + o) * kTileRows + q * 8);
            v0 = __ldg(src);
            v1 = __ldg(src + 1);
        };
        skip_empty_tiles();
        if (tile < active) {
            enter_tile();
            if (a_half < units) {
                load_vector(i0, i1);
            }
        }
        while (tile < active) {
            // ---- what this slab needs ----
            const bool uv = 2 * s + a_half < units;
            const int k = uv ? __ffs(rem) - 1 : 0;
            const int col = (uv ? slice : 0) * 32 + col8;
            const int idx[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
            // ---- step the cursor and prefetch the next slab's row vector ----
            const int prev_o = o;
            bool moved = false;
            ++s;
            if (2 * s < units) {
                slice += 2;
                while (slice >= upo) {
                    slice -= upo;
                    ++o;
                    rem &= rem - 1;
                }
            } else {
                tile += grid;
                info = next_info;
                next_info = load_info(p, tile + grid, active);
                skip_empty_tiles();
                if (tile < active) {
                    enter_tile();
                }
                moved = true;
            }
            int4 n0 = i0, n1 = i1;
            if (tile < active && (moved || o != prev_o) && 2 * s + a_half < units) {
                load_vector(n0, n1);
            }
            // ---- this slab's copies ----
            if (!mbar_wait(&ctl.empty[ring.index], ring.phase ^ 1u, abort_flag, p.status)) {
                ok = false;
                break;
            }
            const uint32_t a_addr = smem_u32(smem + ring.index * p.stage_bytes) + dst0;
            const uint32_t b_addr = a_addr + kSlabBytesA;
            const char* const col_base = feat_bytes + col * 2;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // absent neighbours (and the unused half of an odd last slab) copy zero
                // bytes from a valid address: the destination is zero-filled
                const int in_row = uv ? idx[j] : -1;
                cp_async_16(a_addr + 4096 * j,
                            col_base + static_cast<long long>(max(in_row, 0)) * feat_row_bytes,
                            in_row >= 0);
            }
            if (p.b_tma) {
                // both units of the slab share the offset k: the B tile is one box of
                // C_out rows x 64 channels, fetched by the TMA unit (thread 0's unit is the
                // slab's first, so its k and column are the box origin)
                if (tid == 0) {
                    mbar_arrive_expect_tx(&ctl.full[ring.index], static_cast<uint32_t>(p.c_out) * 128u);
                    tma_load_3d(b_addr - dst0, &b_map, col, p.b_k_outer ? 0 : k, p.b_k_outer ? k : 0,
                                &ctl.full[ring.index]);
                }
            } else {
                const char* w_src =
                    weight_bytes + static_cast<long long>(k) * p.w_k_bytes + col * 2 + w_co0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i < b_copies) {
                        cp_async_16(b_addr + 4096 * i, w_src, uv);
                        w_src += w_co_step;
                    }
                }
                if (p.c_out & 16) {
                    // C_out = 32 m + 16: the last 16 output channels
                    if (q < 16) {
                        cp_async_16(b_addr + 4096 * b_copies, w_src, uv);
                    }
                }
            }
            cp_async_arrive_noinc(&ctl.full[ring.index]);
            ring.advance(p.stages);
            i0 = n0;
            i1 = n1;
        }
        cp_async_wait<0>();
        }
        for (int tile = blockIdx.x + ((active - blockIdx.x + grid - 1) / grid) * grid;
             tile < p.num_tiles; tile += grid) {
            if (producers_fill(tile, grid)) {
                fill_edgeless_rows(p, tile, warp, lane);
            }
        }
    } else if (warp < 16) {
        // ======================= epilogue =======================
        const int ew = warp - 8;
        const int quarter = ew & 3;       // TMEM lanes 32*quarter .. +31 (warp index % 4)
        const int half_tile = ew >> 2;    // which 128-row half of the tile
        const int tile_row = half_tile * 128 + quarter * 32 + lane;
        bool ok = true;
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += grid, ++local_tile) {
            const int position = tile * kTileRows + tile_row;
            int row = -1;
            if (position < p.out_capacity) {
                row = p.row_order != nullptr ? __ldg(p.row_order + position) : position;
                if (row < 0 || row >= p.out_capacity) {
                    raise_status(p.status, LAT_STATUS_BAD_INDEX);
                    row = -1;
                }
            }
            bool computed = false;
            int a = 0;
            if (tile < active) {
                const int2 info = __ldg(p.tile_info + tile);
                a = local_tile % p.acc_stages;
                const uint32_t parity = (local_tile / p.acc_stages) & 1;
                if (!mbar_wait(&ctl.acc_full[a], parity, abort_flag, p.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                computed = info.x != 0;
            }
            __half* out_row = row >= 0 ? p.out + static_cast<size_t>(row) * p.c_out : nullptr;
            if (!computed) {
                if (tile < active || !producers_fill(tile, grid)) {
                    fill_edgeless_rows(p, tile, ew, lane);
                }
                if (tile < active) {
                    tc_fence_before();
                    mbar_arrive(&ctl.acc_empty[a]);
                }
                continue;
            }
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>((2 * a + half_tile) * p.acc_cols);
            for (int c0 = 0; c0 < p.c_out; c0 += 32) {
                uint32_t v[32];
                const int width = min(32, p.c_out - c0);  // 32 or 16
                if (computed) {
                    if (width == 32) {
                        tmem_load_32(taddr + c0, v);
                    } else {
                        tmem_load_16(taddr + c0, v);
                    }
                    tmem_load_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v[i] = 0u;
                    }
                }
                if (out_row != nullptr) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (i < width) {
                            __half2 h[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __half hx = __float2half_rn(__uint_as_float(v[i + 2 * j]));
                                __half hy = __float2half_rn(__uint_as_float(v[i + 2 * j + 1]));
                                if (p.bias != nullptr) {
                                    hx = __float2half_rn(__half2float(hx) +
                                                         __half2float(__ldg(p.bias + c0 + i + 2 * j)));
                                    hy = __float2half_rn(__half2float(hy) +
                                                         __half2float(__ldg(p.bias + c0 + i + 2 * j + 1)));
                                }
                                h[j] = __halves2half2(hx, hy);
                            }
                            *reinterpret_cast<uint4*>(out_row + c0 + i) = *reinterpret_cast<uint4*>(h);
                        }
                    }
                }
            }
            if (tile < active) {
                tc_fence_before();
                mbar_arrive(&ctl.acc_empty[a]);
            }
        }
    } else if (lane == 0) {
        // ======================= MMA issuer =======================
        const uint32_t idesc = make_instr_desc(128, p.c_out);
        bool ok = true;
        Ring ring{0, 0u};
        int local_tile = 0;
        int2 info = load_info(p, blockIdx.x, active);
        for (int tile = blockIdx.x; tile < active && ok; tile += grid, ++local_tile) {
            const int2 next_info = load_info(p, tile + grid, active);
            const int a = local_tile % p.acc_stages;
            const uint32_t parity = (local_tile / p.acc_stages) & 1;
            if (!mbar_wait(&ctl.acc_empty[a], parity ^ 1, abort_flag, p.status)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int slabs = (__popc(static_cast<uint32_t>(info.x)) * upo + 1) >> 1;
            const uint32_t tmem_d0 = tmem_base + static_cast<uint32_t>(2 * a * p.acc_cols);
            const uint32_t tmem_d1 = tmem_d0 + static_cast<uint32_t>(p.acc_cols);
            for (int s = 0; s < slabs; ++s) {
                if (!mbar_wait(&ctl.full[ring.index], ring.phase, abort_flag, p.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + ring.index * p.stage_bytes);
                const uint64_t desc_a0 = make_smem_desc(a_addr);
                const uint64_t desc_a1 = make_smem_desc(a_addr + 128 * 128);
                const uint64_t desc_b = make_smem_desc(a_addr + kSlabBytesA);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    // 16 fp16 = 32 bytes along K inside the swizzle atom: +2 in 16-byte units
                    const uint32_t acc = (s | kk) != 0 ? 1u : 0u;
                    umma_f16(tmem_d0, desc_a0 + 2 * kk, desc_b + 2 * kk, idesc, acc);
                    umma_f16(tmem_d1, desc_a1 + 2 * kk, desc_b + 2 * kk, idesc, acc);
                }
                umma_commit(&ctl.empty[ring.index]);
                ring.advance(p.stages);
            }
            if (!ok) {
                break;
            }
            if (slabs > 0) {
                umma_commit(&ctl.acc_full[a]);
            } else {
                mbar_arrive(&ctl.acc_full[a]);
            }
            info = next_info;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(p.tmem_cols))
                     : "memory");
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
using EncodeTiledFn = CUresult (*)(
    CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) ==
                cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        }
    });
    return fn;
}

int pow2_at_least(int value, int floor_value) {
    int out = floor_value;
    while (out < value) {
        out <<= 1;
    }
    return out;
}

} // namespace

// fp16 weights only (packed weights are staged to fp16 by the caller); shapes as
// tc_conv_supported allows them.
int run_tc_conv_plan(
    const void* feats, int in_channels, long long feat_stride, const void* weights,
    long long w_stride_k, long long w_stride_co, int n_kernels, int out_channels, int out_capacity,
    const void* bias, const int32_t* row_order, const void* plan, void* out, int32_t* status,
    cudaStream_t stream
) {
    if (out_capacity == 0) {
        return LAT_OK;
    }
    PlanConvParams p{};
    p.feats = static_cast<const __half*>(feats);
    LAT_REQUIRE(feat_stride > 0 && feat_stride * 2 < (1LL << 31),
                "feature row stride is out of range for the tensor-core route.");
    p.feat_row_bytes = static_cast<int>(feat_stride * 2);
    p.c_in = in_channels;
    p.c_out = out_channels;
    p.weights = static_cast<const __half*>(weights);
    p.w_k_bytes = w_stride_k * 2;
    p.w_co_bytes = w_stride_co * 2;
    p.num_tiles = plan_tiles(out_capacity);
    p.tile_info = static_cast<const int2*>(plan);
    p.vectors = reinterpret_cast<const int32_t*>(static_cast<const char*>(plan) + plan_info_bytes(p.num_tiles));
    p.row_order = row_order;
    p.out_capacity = out_capacity;
    p.bias = static_cast<const __half*>(bias);
    p.out = static_cast<__half*>(out);
    p.status = status;
    p.acc_cols = pow2_at_least(out_channels, 32);
    p.acc_stages = std::min(kMaxAccStages, 512 / (2 * p.acc_cols));
    p.tmem_cols = p.acc_stages * 2 * p.acc_cols;
    // every B tile on a 1024-byte boundary (the swizzle pattern repeats every eight rows)
    p.stage_bytes = kSlabBytesA + static_cast<int>(align_up(static_cast<size_t>(out_channels) * 128, 1024));
    const int ctl_bytes = static_cast<int>(align_up(sizeof(Control), 16));
    const int smem_budget = 227 * 1024 - 1024 /*alignment slack*/ - ctl_bytes;
    p.stages = std::min(kMaxStages, smem_budget / p.stage_bytes);
    LAT_REQUIRE(p.stages >= 2, "internal: shared-memory plan leaves no room for the stage ring.");
    const size_t smem_bytes = 1024 + static_cast<size_t>(p.stages) * p.stage_bytes + ctl_bytes;

    int device = 0;
    LAT_CUDA_CHECK(cudaGetDevice(&device));
    int sm_count = 0;
    LAT_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    const int grid = std::max(1, std::min(p.num_tiles, sm_count));
    LAT_CUDA_CHECK(cudaFuncSetAttribute(
        tc_conv_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)));
    // B tiles by TMA when a slab's two units share their kernel offset (C_in a multiple of
    // 64): a 3-D map over the fp16 weights with the kernel offset as its own dimension
    CUtensorMap b_map{};
    const bool k_outer = w_stride_k >= w_stride_co;
    if (in_channels % 64 == 0 && encode_tiled_fn() != nullptr &&
        reinterpret_cast<uintptr_t>(weights) % 16 == 0 && n_kernels >= 1) {
        const cuuint64_t dims[3] = {static_cast<cuuint64_t>(in_channels),
                                    static_cast<cuuint64_t>(k_outer ? out_channels : n_kernels),
                                    static_cast<cuuint64_t>(k_outer ? n_kernels : out_channels)};
        const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k_outer ? p.w_co_bytes : p.w_k_bytes),
                                       static_cast<cuuint64_t>(k_outer ? p.w_k_bytes : p.w_co_bytes)};
        const cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(k_outer ? out_channels : 1),
                                   static_cast<cuuint32_t>(k_outer ? 1 : out_channels)};
        const cuuint32_t elem_strides[3] = {1u, 1u, 1u};
        CUresult rc = encode_tiled_fn()(
            &b_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(weights), dims, strides, box,
            elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc == CUDA_SUCCESS) {
            p.b_tma = 1;
            p.b_k_outer = k_outer ? 1 : 0;
        }
    }
    tc_conv_plan_kernel<<<grid, kThreads, smem_bytes, stream>>>(p, b_map);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // namespace lat

// Tensor-core sparse convolution driven by a gather plan (conv_plan.cu): an output-stationary
// implicit GEMM on tcgen05 -- 256-row tiles of output rows in the plan's row order, a unit =
// (kernel offset used by the tile, 32-channel slice of C_in), two units per 64-wide K slab,
// fp32 accumulators in TMEM, one deterministic store per output row. The persistent CTAs take
// the tiles in the plan's tile order (tiles by falling number of used offsets) in a
// serpentine, so that each of them gets about the same number of slabs; every role of a CTA
// computes that sequence for itself. No role touches the relation's CSR arrays and no
// thread waits for a copy of its own:
//   warp 17    row-vector loader: streams the plan's row vectors of the CTA's tiles (one
//              per tile and used kernel offset, 1 KB each) into a 16-slot shared-memory
//              ring by bulk copies, in the order the producers consume them, so that no
//              producer waits on a global load of the plan.
//   warps 0-7  producers. A thread owns one 16-byte chunk column (so one unit of each
//              slab) and the eight tile rows q, q+32, ..; their input rows are 32
//              contiguous bytes of a row vector in the ring. Per slab: wait for a free
//              stage, 8 cp.async for A (zero fill where the row has no neighbour; the
//              channels may come from two feature tensors over the same rows), the fp16
//              B tile, then cp.async.mbarrier.arrive.noinc so that the stage's barrier
//              completes when the copies land. The stream of slabs runs across tile
//              boundaries. When C_in is a multiple of 64 both units of a slab share
//              their kernel offset: one ring entry feeds C_in / 64 slabs and the weight
//              tile of a slab is one TMA box (cp.async.bulk.tensor.3d, 128-byte swizzle,
//              no multicast) issued by one thread.
//   warp 16    one thread issues the MMAs (8 per slab), commits the stage back to the
//              producers and, per tile, the accumulator to the epilogue.
//   warps 8-15 epilogue: tcgen05.ld, optional bias, one cast to fp16, 32-byte stores.
// Every mbarrier wait is bounded by a clock budget (lat_set_wait_budget_cycles) and its
// verdict is made uniform across the warp; on expiry the kernel records
// LAT_STATUS_WAIT_TIMEOUT, every role leaves its loop, the CTA lets copies in flight land
// and frees its TMEM.
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
constexpr int kProducerWarps = 8;

constexpr int kVectorRing = 16;                   // most row vectors held in shared memory
constexpr int kVectorBytes = kPlanTileRows * 4;
constexpr int kMaxStages = 8;
constexpr int kMaxAccStages = 8;
constexpr int kSlabBytesA = kTileRows * 128;

struct PlanConvParams {
    // Feature rows may come from two tensors over the same rows: channels [0, split) from
    // `feats`, channels [split, c_in) from `feats2` (the concatenation of a decoder level
    // read in place). split == c_in when there is one source. split is a multiple of 8.
    const __half* feats;
    const __half* feats2;
    int feat_row_bytes;
    int feat2_row_bytes;
    int split;
    int c_in;
    int c_out;
    // fp16 weights addressed (in bytes) as base + k*w_k_bytes + co*w_co_bytes + 2*ci
    const __half* weights;
    long long w_k_bytes;
    long long w_co_bytes;
    const int2* tile_info;     // [num_tiles + 1]; the last entry holds (tiles in use, vectors)
    const int32_t* tile_order; // [num_tiles]: tiles by falling number of used offsets
    const int32_t* vectors;
    const int32_t* row_order;
    int out_capacity;
    const __half* bias;
    __half* out;
    int32_t* status;
    long long wait_budget;
    int stages;
    int vec_slots;       // row vectors in the shared-memory ring (at most kVectorRing)
    int stage_bytes;     // 32 KB of A rows + the B tile
    int tmem_cols;
    int acc_cols;
    int acc_stages;
    int num_tiles;
    int wide_stores;     // 1: `out` is 32-byte aligned and rows are stored 32 bytes at a time
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
    uint64_t vec_full[kVectorRing];
    uint64_t vec_empty[kVectorRing];
    int32_t vec_header[kVectorRing];
    uint32_t tmem_base;
    int abort_flag;
};

// header of a row vector in the shared-memory ring: kernel offset, position inside the
// tile and how many vectors the tile has; negative = no more work for this CTA
__device__ __forceinline__ int32_t make_header(int k, int present) { return k | (present << 8); }
__device__ __forceinline__ int header_k(int32_t h) { return h & 31; }
__device__ __forceinline__ int header_present(int32_t h) { return (h >> 8) & 63; }

// The turn-th tile of CTA `cta`: the CTAs walk the plan's tile order (tiles by falling cost)
// in a serpentine, so that every pair of rounds hands each of them about the same work.
// -1 at and beyond position `limit`; positions grow with the turn.
__device__ __forceinline__ int tile_of_turn(const PlanConvParams& p, int turn, int cta, int grid, int limit) {
    const int position = plan_position(turn, cta, grid);
    return position < limit ? __ldg(p.tile_order + position) : -1;
}

__device__ __forceinline__ int2 load_info(const PlanConvParams& p, int tile) {
    return tile >= 0 ? __ldg(p.tile_info + tile) : make_int2(0, 0);
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

// Sixteen fp16 values as one 32-byte store (dst 32-byte aligned): each lane of the epilogue
// writes its own output row, so a 16-byte store fills half a 32-byte sector and the row's
// next 16 bytes arrive as a second request; whole sectors halve the requests.
__device__ __forceinline__ void store_f16x16(__half* dst, const uint4& lo, const uint4& hi) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(lo.x), "r"(lo.y),
                 "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                 : "memory");
}

// the tiles without an edge (the end of the tile order) are shared between the producer
// warps (which run out of work first) and the epilogue warps: even and odd rounds over them
__device__ __forceinline__ bool producers_fill(int index, int grid) { return ((index / grid) & 1) == 0; }

// kEpilogueWarps = 8: one CTA per SM, a warp per 32-row quarter of each 128-row half (C_out
// above 128, where one tile's accumulators fill the tensor memory). kEpilogueWarps = 4: TWO
// CTAs per SM, each with half the stages, half the tensor memory and four epilogue warps
// that take both halves in turn; while one CTA's MMA thread is between slabs (barrier
// test, proxy fence, commit) the other's MMAs keep the pipe busy.
template <int kEpilogueWarps>
__global__ void __launch_bounds__((kProducerWarps + kEpilogueWarps + 2) * 32, kEpilogueWarps == 4 ? 2 : 1)
tc_conv_plan_kernel(PlanConvParams p, const __grid_constant__ CUtensorMap b_map) {
    constexpr int kMmaWarp = kProducerWarps + kEpilogueWarps;
    constexpr int kLoaderWarp = kMmaWarp + 1;
    constexpr int kHalves = 8 / kEpilogueWarps;    // 128-row halves of a tile per epilogue warp
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* const vec_ring = smem + p.stages * p.stage_bytes;
    Control& ctl = *reinterpret_cast<Control*>(vec_ring + p.vec_slots * kVectorBytes);
    volatile int* abort_flag = &ctl.abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int upo = p.c_in / 32;  // units per kernel offset
    const int grid = gridDim.x;
    const long long budget = p.wait_budget;
    // Bounded wait whose verdict is the same in every lane of the (converged) warp, so that a
    // wait that gives up takes the whole warp out of its loop and no lane is left behind at
    // a warp-level synchronisation.
    auto wait_warp = [&](uint64_t* bar, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, p.status, budget));
    };

    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl.full[s], kProducerWarps * 32 + (p.b_tma ? 1 : 0));
            mbar_init(&ctl.empty[s], 1);
        }
        for (int a = 0; a < kMaxAccStages; ++a) {
            mbar_init(&ctl.acc_full[a], 1);
            mbar_init(&ctl.acc_empty[a], kEpilogueWarps);
        }
        for (int v = 0; v < kVectorRing; ++v) {
            mbar_init(&ctl.vec_full[v], 1);
            mbar_init(&ctl.vec_empty[v], kProducerWarps);
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
    // positions [0, used) of the tile order hold the tiles that use a kernel offset, the
    // rest use none at all
    const int used = min(max(__ldg(&p.tile_info[p.num_tiles].x), 0), p.num_tiles);
    const int idle = p.num_tiles - used;

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
        const char* const weight_bytes = reinterpret_cast<const char*>(p.weights);
        const long long w_co0 = static_cast<long long>(q) * p.w_co_bytes;
        const long long w_co_step = 32LL * p.w_co_bytes;
        const int b_copies = p.c_out >> 5;  // C_out is a multiple of 32 here, or 16 (see below)
        // byte address and row pitch of channel `channel` of row 0 in the tensor that holds it
        auto channel_base = [&](int channel, int& pitch) -> const char* {
            if (channel < p.split) {
                pitch = p.feat_row_bytes;
                return reinterpret_cast<const char*>(p.feats) + channel * 2;
            }
            pitch = p.feat2_row_bytes;
            return reinterpret_cast<const char*>(p.feats2) + (channel - p.split) * 2;
        };
        // this thread's eight row ids of a vector in the ring (32 contiguous bytes)
        auto read_vector = [&](int slot, int4& d0, int4& d1) {
            const uint32_t src = smem_u32(vec_ring + slot * kVectorBytes + q * 32);
            d0 = lds_v4_pinned(src);
            d1 = lds_v4_pinned(src + 16);
        };
        Ring ring{0, 0u};
        Ring vec{0, 0u};
        bool ok = true;
        // wait for stage `ring.index` to be free (the warp decides as one)
        auto acquire_stage = [&]() -> bool {
            const bool got = wait_warp(&ctl.empty[ring.index], ring.phase ^ 1u);
            return got;
        };
        // The slab in stage `ring.index` is issued. Every thread's copies arrive on the stage's
        // barrier by themselves when they have landed (no thread waits for its own copies).
        auto slab_issued = [&]() {
            cp_async_arrive_noinc(&ctl.full[ring.index]);
            ring.advance(p.stages);
        };

        if ((upo & 1) == 0) {
            // ---- C_in a multiple of 64: both units of a slab belong to one kernel offset ----
            // One ring entry = one (tile, offset) = C_in / 64 slabs. Tile boundaries do not
            // matter here: the stream of slabs runs on until the loader's end marker.
            const int reps = upo >> 1;  // slabs per offset
            const int thread_channel = a_half * 32 + col8;
            while (ok) {
                if (!wait_warp(&ctl.vec_full[vec.index], vec.phase)) {
                    ok = false;
                    break;
                }
                const int32_t header = ctl.vec_header[vec.index];
                if (header < 0) {
                    break;
                }
                int4 v0, v1;
                read_vector(vec.index, v0, v1);
                const int k = header_k(header);
                const int idx[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                for (int r = 0; r < reps; ++r) {
                    int pitch;
                    const char* const base = channel_base(r * 64 + thread_channel, pitch);
                    if (!acquire_stage()) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_addr = smem_u32(smem + ring.index * p.stage_bytes) + dst0;
                    const uint32_t b_addr = a_addr + kSlabBytesA;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // absent neighbours copy zero bytes from a valid address: zero fill
                        cp_async_16(a_addr + 4096 * j,
                                    base + static_cast<long long>(max(idx[j], 0)) * pitch, idx[j] >= 0);
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
                                            r * 128 + thread_channel * 2 + w_co0;
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
                    slab_issued();
                    if (r == 0) {
                        // The slot goes back to the loader only now: the copies above took
                        // their addresses from the row ids, so every lane's reads of the slot
                        // have returned before it can be overwritten.
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive(&ctl.vec_empty[vec.index]);
                        }
                        vec.advance(p.vec_slots);
                    }
                }
            }
        } else {
            // ---- general case: a slab may straddle two kernel offsets ----
            // Unit u of a tile = (offset u / upo, 32-channel slice u % upo); slab s holds the
            // units 2 s and 2 s + 1, this thread feeds unit 2 s + a_half. Ring entries are
            // released in order once no later slab of any thread needs them: before slab s,
            // everything below the entry of unit 2 s.
            Ring released{0, 0u};   // next entry this thread has not released yet
            auto release_until = [&](int count) -> bool {
                for (int i = 0; i < count; ++i) {
                    if (!wait_warp(&ctl.vec_full[released.index], released.phase)) {
                        return false;
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&ctl.vec_empty[released.index]);
                    }
                    released.advance(p.vec_slots);
                }
                return true;
            };
            while (ok) {
                // `vec` is the first entry of the tile
                if (!wait_warp(&ctl.vec_full[vec.index], vec.phase)) {
                    ok = false;
                    break;
                }
                const int32_t first = ctl.vec_header[vec.index];
                if (first < 0) {
                    break;
                }
                const int present = header_present(first);
                const int units = present * upo;
                const int slabs = (units + 1) >> 1;
                int done = 0;        // entries of this tile already released
                int held = -1;       // offset position whose row ids sit in v0, v1
                int k = 0;
                int4 v0 = make_int4(-1, -1, -1, -1), v1 = v0;
                for (int s = 0; s < slabs && ok; ++s) {
                    const int u = 2 * s + a_half;
                    const bool uv = u < units;
                    const int o = uv ? u / upo : 0;
                    const int slice = u - o * upo;
                    const int o_low = (2 * s) / upo;
                    if (!release_until(o_low - done)) {
                        ok = false;
                        break;
                    }
                    done = o_low;
                    {
                        // The entry this lane reads (the lanes of the unused half of an odd
                        // last slab wait on the slab's first entry, so that the whole warp
                        // waits and decides together): up to two trips round the ring away.
                        const int position = vec.index + (uv ? o : o_low);
                        const int slot = position % p.vec_slots;
                        const uint32_t phase = vec.phase ^ static_cast<uint32_t>((position / p.vec_slots) & 1);
                        if (!wait_warp(&ctl.vec_full[slot], phase)) {
                            ok = false;
                            break;
                        }
                        if (uv && o != held) {
                            k = header_k(ctl.vec_header[slot]);
                            read_vector(slot, v0, v1);
                            held = o;
                        }
                    }
                    const int idx[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    const int channel = (uv ? slice : 0) * 32 + col8;
                    int pitch;
                    const char* const base = channel_base(channel, pitch);
                    if (!acquire_stage()) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_addr = smem_u32(smem + ring.index * p.stage_bytes) + dst0;
                    const uint32_t b_addr = a_addr + kSlabBytesA;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // absent neighbours (and the unused half of an odd last slab) copy zero
                        // bytes from a valid address: the destination is zero-filled
                        const int in_row = uv ? idx[j] : -1;
                        cp_async_16(a_addr + 4096 * j,
                                    base + static_cast<long long>(max(in_row, 0)) * pitch, in_row >= 0);
                    }
                    const char* w_src = weight_bytes + static_cast<long long>(uv ? k : 0) * p.w_k_bytes +
                                        channel * 2 + w_co0;
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
                    slab_issued();
                }
                if (ok && !release_until(present - done)) {
                    ok = false;
                }
                for (int i = 0; i < present; ++i) {
                    vec.advance(p.vec_slots);
                }
            }
        }
        cp_async_wait<0>();
        for (int index = blockIdx.x; index < idle; index += grid) {
            if (producers_fill(index, grid)) {
                fill_edgeless_rows(p, __ldg(p.tile_order + used + index), warp, lane);
            }
        }
    } else if (warp < kMmaWarp) {
        // ======================= epilogue =======================
        const int ew = warp - kProducerWarps;
        const int quarter = ew & 3;       // TMEM lanes 32*quarter .. +31 (warp index % 4)
        const int first_half = kHalves == 1 ? ew >> 2 : 0;   // the 128-row halves this warp stores
        bool ok = true;
        int local_tile = 0;
        // the output rows of a tile are fetched one tile ahead
        auto tile_output_row = [&](int tile, int half_tile) -> int {
            const int position = tile * kTileRows + half_tile * 128 + quarter * 32 + lane;
            if (tile < 0 || position >= p.out_capacity) {
                return -1;
            }
            return p.row_order != nullptr ? __ldg(p.row_order + position) : position;
        };
        int next_tile = tile_of_turn(p, 0, blockIdx.x, grid, used);
        int next_row[kHalves];
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
            next_row[h] = tile_output_row(next_tile, first_half + h);
        }
        for (int turn = 0; next_tile >= 0 && ok; ++turn, ++local_tile) {
            const int tile = next_tile;
            next_tile = tile_of_turn(p, turn + 1, blockIdx.x, grid, used);
            int rows[kHalves];
#pragma unroll
            for (int h = 0; h < kHalves; ++h) {
                rows[h] = next_row[h];
                next_row[h] = tile_output_row(next_tile, first_half + h);
                const int position = tile * kTileRows + (first_half + h) * 128 + quarter * 32 + lane;
                if (rows[h] >= p.out_capacity || (rows[h] < 0 && position < p.out_capacity)) {
                    raise_status(p.status, LAT_STATUS_BAD_INDEX);
                    rows[h] = -1;
                }
            }
            const int a = local_tile % p.acc_stages;
            const uint32_t parity = (local_tile / p.acc_stages) & 1;
            if (!wait_warp(&ctl.acc_full[a], parity)) {
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < kHalves; ++h) {
                const int half_tile = first_half + h;
                __half* out_row = rows[h] >= 0 ? p.out + static_cast<size_t>(rows[h]) * p.c_out : nullptr;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>((2 * a + half_tile) * p.acc_cols);
                for (int c0 = 0; c0 < p.c_out; c0 += 32) {
                    uint32_t v[32];
                    const int width = min(32, p.c_out - c0);  // 32 or 16
                    if (width == 32) {
                        tmem_load_32(taddr + c0, v);
                    } else {
                        tmem_load_16(taddr + c0, v);
                    }
                    tmem_load_wait();
                    if (out_row != nullptr) {
#pragma unroll
                        for (int i = 0; i < 32; i += 16) {
                            if (i < width) {
                                __half2 pair[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    __half hx = __float2half_rn(__uint_as_float(v[i + 2 * j]));
                                    __half hy = __float2half_rn(__uint_as_float(v[i + 2 * j + 1]));
                                    if (p.bias != nullptr) {
                                        hx = __float2half_rn(__half2float(hx) +
                                                             __half2float(__ldg(p.bias + c0 + i + 2 * j)));
                                        hy = __float2half_rn(__half2float(hy) +
                                                             __half2float(__ldg(p.bias + c0 + i + 2 * j + 1)));
                                    }
                                    pair[j] = __halves2half2(hx, hy);
                                }
                                const uint4 lo = *reinterpret_cast<uint4*>(pair);
                                const uint4 hi = *reinterpret_cast<uint4*>(pair + 4);
                                __half* const dst = out_row + c0 + i;
                                if (p.wide_stores) {
                                    store_f16x16(dst, lo, hi);
                                } else {
                                    *reinterpret_cast<uint4*>(dst) = lo;
                                    *reinterpret_cast<uint4*>(dst + 8) = hi;
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl.acc_empty[a]);
            }
        }
        // this role's share of the tiles without an edge
        for (int index = blockIdx.x; index < idle && ok; index += grid) {
            if (!producers_fill(index, grid)) {
                const int tile = __ldg(p.tile_order + used + index);
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    fill_edgeless_rows(p, tile, (first_half + h) * 4 + quarter, lane);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ======================= MMA issuer =======================
        // Lane 0 issues; the warp as a whole fetches the offset masks of the CTA's next 32
        // tiles in one load each, a batch ahead of their use.
        const uint32_t idesc = make_instr_desc(128, p.c_out);
        const uint64_t desc0 = make_smem_desc(smem_u32(smem));
        const uint32_t desc_lo0 = static_cast<uint32_t>(desc0);
        const uint32_t desc_hi = static_cast<uint32_t>(desc0 >> 32);
        const uint32_t stage_step = static_cast<uint32_t>(p.stage_bytes) >> 4;
        bool ok = true;
        Ring ring{0, 0u};
        int local_tile = 0;
        int2 batch = load_info(p, tile_of_turn(p, lane, blockIdx.x, grid, used));
        for (int first = 0; ok; first += 32) {
            const int2 mine = batch;   // masks of turns first .. first + 31 (0 past the end)
            batch = load_info(p, tile_of_turn(p, first + 32 + lane, blockIdx.x, grid, used));
            const int count = __popc(__ballot_sync(0xffffffffu, mine.x != 0));
            for (int j = 0; j < count && ok; ++j, ++local_tile) {
                const int mask = __shfl_sync(0xffffffffu, mine.x, j);
                if (lane == 0) {
                    const int a = local_tile % p.acc_stages;
                    const uint32_t parity = (local_tile / p.acc_stages) & 1;
                    if (!mbar_wait(&ctl.acc_empty[a], parity ^ 1, abort_flag, p.status, budget)) {
                        ok = false;
                    }
                    tc_fence_after();
                    const int slabs = (__popc(static_cast<uint32_t>(mask)) * upo + 1) >> 1;
                    const uint32_t tmem_d0 = tmem_base + static_cast<uint32_t>(2 * a * p.acc_cols);
                    const uint32_t tmem_d1 = tmem_d0 + static_cast<uint32_t>(p.acc_cols);
                    for (int s = 0; s < slabs && ok; ++s) {
                        if (!mbar_wait(&ctl.full[ring.index], ring.phase, abort_flag, p.status, budget)) {
                            ok = false;
                            break;
                        }
                        // the A rows were written by cp.async (generic proxy); the MMA reads
                        // shared memory through the async proxy
                        fence_proxy_async();
                        tc_fence_after();
                        // descriptors of the stage's operands: the address field is the low
                        // 14 bits of the low word (16-byte units), everything else is fixed
                        const uint32_t a_lo = desc_lo0 + static_cast<uint32_t>(ring.index) * stage_step;
                        const uint32_t b_lo = a_lo + (kSlabBytesA >> 4);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            // 16 fp16 = 32 bytes along K inside the swizzle atom: +2 in 16-byte units
                            const uint32_t acc = kk != 0 ? 1u : (s != 0 ? 1u : 0u);
                            umma_f16_split(tmem_d0, a_lo + 2 * kk, b_lo + 2 * kk, desc_hi, idesc, acc);
                            umma_f16_split(tmem_d1, a_lo + (128 * 128 >> 4) + 2 * kk, b_lo + 2 * kk, desc_hi,
                                           idesc, acc);
                        }
                        umma_commit(&ctl.empty[ring.index]);
                        ring.advance(p.stages);
                    }
                    if (ok) {
                        if (slabs > 0) {
                            umma_commit(&ctl.acc_full[a]);
                        } else {
                            mbar_arrive(&ctl.acc_full[a]);
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (count < 32) {
                break;
            }
        }
    } else if (warp == kLoaderWarp) {
        // ======================= row-vector loader =======================
        // Streams the row vectors of this CTA's tiles, in the order the producers consume
        // them, into a shared-memory ring by bulk copies, so that no producer ever waits on
        // a global load of the plan. Lane 0 issues; the warp fetches offset masks in batches.
        bool ok = true;
        Ring vec{0, 0u};
        auto publish = [&](int32_t header, const int32_t* source) -> bool {
            if (!mbar_wait(&ctl.vec_empty[vec.index], vec.phase ^ 1u, abort_flag, p.status, budget)) {
                return false;
            }
            ctl.vec_header[vec.index] = header;
            if (source != nullptr) {
                mbar_arrive_expect_tx(&ctl.vec_full[vec.index], kVectorBytes);
                bulk_load(smem_u32(vec_ring + vec.index * kVectorBytes), source, kVectorBytes,
                          &ctl.vec_full[vec.index]);
            } else {
                mbar_arrive(&ctl.vec_full[vec.index]);
            }
            vec.advance(p.vec_slots);
            return true;
        };
        int2 batch = load_info(p, tile_of_turn(p, lane, blockIdx.x, grid, used));
        for (int first = 0; ok; first += 32) {
            const int2 mine = batch;
            batch = load_info(p, tile_of_turn(p, first + 32 + lane, blockIdx.x, grid, used));
            const int count = __popc(__ballot_sync(0xffffffffu, mine.x != 0));
            for (int j = 0; j < count && ok; ++j) {
                const int mask = __shfl_sync(0xffffffffu, mine.x, j);
                const int vector0 = __shfl_sync(0xffffffffu, mine.y, j);
                if (lane == 0) {
                    uint32_t rem = static_cast<uint32_t>(mask);
                    const int present = __popc(rem);
                    for (int o = 0; o < present && ok; ++o) {
                        const int k = __ffs(rem) - 1;
                        rem &= rem - 1;
                        ok = publish(make_header(k, present),
                                     p.vectors + (static_cast<size_t>(vector0) + o) * kTileRows);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (count < 32) {
                break;
            }
        }
        if (lane == 0 && ok) {
            publish(-1, nullptr);
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (ctl.abort_flag != 0) {
        // a role gave up: bulk copies towards this CTA's shared memory may still be in flight;
        // they land within microseconds, and the CTA stays until they have
        const long long start = clock64();
        while (clock64() - start < 200000) {
        }
        __syncthreads();
    }
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
// tc_conv_supported allows them. `feats2` (optional) holds the channels from `split` on.
int run_tc_conv_plan(
    const void* feats, int in_channels, long long feat_stride, const void* feats2, int split,
    long long feat2_stride, const void* weights,
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
    if (feats2 != nullptr) {
        LAT_REQUIRE(split > 0 && split < in_channels && split % 8 == 0,
                    "the channel split of a two-source convolution must be a multiple of 8 inside (0, C_in).");
        LAT_REQUIRE(feat2_stride >= in_channels - split && feat2_stride % 8 == 0 &&
                        feat2_stride * 2 < (1LL << 31) && reinterpret_cast<uintptr_t>(feats2) % 16 == 0,
                    "second feature source must have 16-byte aligned rows of at least C_in - split channels.");
        p.feats2 = static_cast<const __half*>(feats2);
        p.feat2_row_bytes = static_cast<int>(feat2_stride * 2);
        p.split = split;
    } else {
        p.feats2 = p.feats;
        p.feat2_row_bytes = p.feat_row_bytes;
        p.split = in_channels;
    }
    p.c_in = in_channels;
    p.c_out = out_channels;
    p.weights = static_cast<const __half*>(weights);
    p.w_k_bytes = w_stride_k * 2;
    p.w_co_bytes = w_stride_co * 2;
    p.num_tiles = plan_tiles(out_capacity);
    p.tile_info = static_cast<const int2*>(plan);
    p.tile_order = reinterpret_cast<const int32_t*>(static_cast<const char*>(plan) + plan_info_bytes(p.num_tiles));
    p.vectors = reinterpret_cast<const int32_t*>(static_cast<const char*>(plan) + plan_vectors_offset(p.num_tiles));
    LAT_REQUIRE(reinterpret_cast<uintptr_t>(p.vectors) % 16 == 0, "plan must be a 16-byte aligned device buffer.");
    p.row_order = row_order;
    p.out_capacity = out_capacity;
    p.bias = static_cast<const __half*>(bias);
    p.out = static_cast<__half*>(out);
    p.status = status;
    // C_out is a multiple of 16, so every row starts on a 32-byte boundary when `out` does
    p.wide_stores = reinterpret_cast<uintptr_t>(out) % 32 == 0 ? 1 : 0;
    p.wait_budget = wait_budget_cycles();
    p.acc_cols = pow2_at_least(out_channels, 32);
    // every B tile on a 1024-byte boundary (the swizzle pattern repeats every eight rows)
    p.stage_bytes = kSlabBytesA + static_cast<int>(align_up(static_cast<size_t>(out_channels) * 128, 1024));
    const int ctl_bytes = static_cast<int>(align_up(sizeof(Control), 16));
    // Two CTAs per SM where two tiles' accumulators fit half of the tensor memory (C_out up to
    // 128): each gets half of the SM's shared memory (228 KB less 1 KB per CTA that the system
    // keeps) and of its 512 TMEM columns. Otherwise one CTA with everything.
    bool paired = out_channels <= 128;
    int smem_per_cta = paired ? (228 * 1024) / 2 - 1024 : 227 * 1024;
    p.vec_slots = paired ? kVectorRing / 2 : kVectorRing;
    int budget = smem_per_cta - 1024 /*alignment slack*/ - p.vec_slots * kVectorBytes - ctl_bytes;
    if (paired && budget / p.stage_bytes < 2) {
        paired = false;
        smem_per_cta = 227 * 1024;
        p.vec_slots = kVectorRing;
        budget = smem_per_cta - 1024 - p.vec_slots * kVectorBytes - ctl_bytes;
    }
    const int tmem_budget = paired ? 256 : 512;
    p.acc_stages = std::min(kMaxAccStages, tmem_budget / (2 * p.acc_cols));
    p.tmem_cols = p.acc_stages * 2 * p.acc_cols;
    p.stages = std::min(kMaxStages, budget / p.stage_bytes);
    LAT_REQUIRE(p.stages >= 2 && p.acc_stages >= 1,
                "internal: shared-memory plan leaves no room for the stage ring.");
    const size_t smem_bytes =
        1024 + static_cast<size_t>(p.stages) * p.stage_bytes + p.vec_slots * kVectorBytes + ctl_bytes;

    int device = 0;
    LAT_CUDA_CHECK(cudaGetDevice(&device));
    int sm_count = 0;
    LAT_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    const int grid = std::max(1, std::min(p.num_tiles, (paired ? 2 : 1) * sm_count));
    auto kernel = paired ? tc_conv_plan_kernel<4> : tc_conv_plan_kernel<8>;
    const int threads = (kProducerWarps + (paired ? 4 : 8) + 2) * 32;
    LAT_CUDA_CHECK(cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)));
    LAT_CUDA_CHECK(cudaFuncSetAttribute(
        kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
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
    kernel<<<grid, threads, smem_bytes, stream>>>(p, b_map);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // namespace lat

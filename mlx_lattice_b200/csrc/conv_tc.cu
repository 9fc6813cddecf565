// Tensor-core route of the sparse-conv contraction that walks the relation itself (the
// plan-driven kernel in conv_tc_plan.cu is the default when a gather plan exists; this
// one serves calls without a plan and the in-register dequantisation route): an
// output-stationary implicit GEMM on tcgen05 with the accumulator in tensor memory.
//
// One persistent CTA per SM walks 256-row output tiles (rows taken through an
// optional permutation). For a tile the implicit GEMM is
//     D[256, C_out] = sum over units u of  A_u[256, 32] * B_u[32, C_out]
// where a unit is (kernel offset k present in the tile, 32-channel slice h of C_in),
// A_u holds the gathered feature rows X[in_row(r, k), 32h .. 32h+31] (zero where the
// output row has no neighbour at k) and B_u the matching weight slice. Two units make
// one 64-wide K slab = one pipeline stage: A is [256 rows][128 B], B is [C_out rows]
// [128 B], both K-major with the 128-byte swizzle that tcgen05 shared-memory
// descriptors name, so a slab is eight M128 x N(C_out) x K16 tcgen05.mma instructions
// (two row halves share every B slab, which halves the weight work per flop).
// Offsets that no row of the tile uses are skipped entirely.
//
// Warp roles (544 threads):
//   warps 0-7  producers: read the tile's CSR rows into a [256][K] neighbour table,
//              gather A with 16-byte cp.async (zero-fill for absent neighbours) and
//              fill B. fp16 weights: cp.async into the same stage as the A rows, and
//              the copies arrive on the stage's barrier themselves when they land
//              (cp.async.mbarrier.arrive.noinc). Packed int4/int8 codes: loaded one
//              slab ahead into registers, dequantised there (code*scale + bias),
//              stored to a second ring and published after a generic->async proxy
//              fence.
//   warps 8-15 epilogue: tcgen05.ld the fp32 accumulator (lane = tile row), add the
//              optional bias, cast once to fp16 and store each output row exactly once
//              (no atomics, deterministic).
//   warp 16    TMEM allocation and the single MMA-issuing thread.
// The accumulator is a ring of up to eight TMEM stages (512 columns / 2 C_out), so the
// epilogue of a tile overlaps the MMAs of the following ones. Every mbarrier wait is
// bounded by a clock budget; on expiry the kernel records LAT_STATUS_WAIT_TIMEOUT, all
// roles drain and the CTA frees its TMEM.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "tcgen05.cuh"

namespace lat {

using namespace tcgen05;

namespace {

constexpr int kTileRows = 256;
constexpr int kProducerThreads = 256;
constexpr int kEpilogueThreads = 256;
constexpr int kThreads = 544;
constexpr int kMmaWarp = 16;
constexpr int kMaxKernel = 32;
constexpr int kMaxStages = 8;
constexpr int kMaxTasks = 8;   // B chunks per producer thread and slab (C_out <= 256)
constexpr int kMaxAccStages = 8;
constexpr int kSlabBytesA = kTileRows * 128;

struct TcParams {
    const __half* feats;
    long long feat_stride;
    int in_capacity;
    int c_in;
    int c_out;
    int n_kernels;
    // fp16 weights addressed as base + k*w_stride_k + co*w_stride_co + ci
    const __half* weights;
    long long w_stride_k;
    long long w_stride_co;
    // packed weights
    const uint32_t* packed;
    const __half* scales;
    const __half* qbiases;
    int words;       // uint32 words per (k, co)
    int groups;
    int group_size;
    const int32_t* in_rows;
    const int32_t* kernel_ids;
    const int32_t* row_offsets;
    const int32_t* counts;
    int edge_capacity;
    int out_capacity;
    const __half* bias;
    const int32_t* row_order;
    __half* out;
    int32_t* status;
    int a_stages;        // ring of gathered A slabs (32 KB each)
    int b_stages;        // ring of B slabs (c_out * 128 bytes each)
    int b_stage_bytes;
    int a_stage_bytes;   // 32 KB, plus the B tile when A and B share a stage (fp16 weights)
    int tmem_cols;       // allocated columns (power of two >= 32)
    int acc_cols;        // columns per accumulator stage
    int acc_stages;      // accumulator stages in TMEM (power of two)
    int num_tiles;
    int nbr_stride;      // odd stride (in ints) of the neighbour table rows
    int ctl_bytes;
};

// ---- in-register dequantisation --------------------------------------------------

// eight int4 codes of one word (channel i in nibble i) -> eight fp16 values
// code*scale + bias, written as one 16-byte vector in channel order
__device__ __forceinline__ uint4 dequant_int4(uint32_t word, __half2 scale, __half2 bias) {
    const uint32_t magic = 0x64006400u;  // fp16 1024.0 in both halves
    const __half2 k1024 = __halves2half2(__ushort_as_half(0x6400), __ushort_as_half(0x6400));
    uint32_t raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // halves: (nibble i, nibble i + 4), each as 1024 + code
        raw[i] = ((word >> (4 * i)) & 0x000F000Fu) | magic;
    }
    __half2 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 code = __hsub2(*reinterpret_cast<__half2*>(&raw[i]), k1024);
        v[i] = __hfma2(code, scale, bias);
    }
    uint32_t a = *reinterpret_cast<uint32_t*>(&v[0]);
    uint32_t b = *reinterpret_cast<uint32_t*>(&v[1]);
    uint32_t c = *reinterpret_cast<uint32_t*>(&v[2]);
    uint32_t d = *reinterpret_cast<uint32_t*>(&v[3]);
    uint4 out;
    out.x = __byte_perm(a, b, 0x5410);  // channels 0, 1
    out.y = __byte_perm(c, d, 0x5410);  // channels 2, 3
    out.z = __byte_perm(a, b, 0x7632);  // channels 4, 5
    out.w = __byte_perm(c, d, 0x7632);  // channels 6, 7
    return out;
}

// four int8 codes of one word (channel i in byte i) -> four fp16 values (8 bytes)
__device__ __forceinline__ uint2 dequant_int8(uint32_t word, __half2 scale, __half2 bias) {
    const __half2 k1024 = __halves2half2(__ushort_as_half(0x6400), __ushort_as_half(0x6400));
    uint32_t lo = __byte_perm(word, 0x64646464u, 0x4140);  // (1024 + b0, 1024 + b1)
    uint32_t hi = __byte_perm(word, 0x64646464u, 0x4342);  // (1024 + b2, 1024 + b3)
    __half2 v0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&lo), k1024), scale, bias);
    __half2 v1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&hi), k1024), scale, bias);
    uint2 out;
    out.x = *reinterpret_cast<uint32_t*>(&v0);
    out.y = *reinterpret_cast<uint32_t*>(&v1);
    return out;
}

// ---- the kernel ---------------------------------------------------------------

// Ring position kept incrementally: runtime divisions are far too slow for the
// per-slab loops (they run on the special-function pipe).
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

// Position in the unit list of a tile: unit = (klist[offset], slice) with `per_offset`
// 32-channel slices per kernel offset.
struct UnitCursor {
    int unit;
    int offset;
    int slice;
    __device__ __forceinline__ void advance(int n, int per_offset) {
        unit += n;
        slice += n;
        while (slice >= per_offset) {
            slice -= per_offset;
            ++offset;
        }
    }
};

// Fixed part of the control block; tile_rows[acc_stages][256] and the neighbour table
// [256][nbr_stride] follow it in shared memory.
struct SharedControl {
    uint64_t full_a[kMaxStages];   // A rows (and the fp16 B tile) of a stage landed
    uint64_t full_b[kMaxStages];   // converted B tile of a stage is written
    uint64_t a_empty[kMaxStages];
    uint64_t b_empty[kMaxStages];
    uint64_t info_full[kMaxAccStages];
    uint64_t acc_full[kMaxAccStages];
    uint64_t acc_empty[kMaxAccStages];
    uint32_t tmem_base;
    int abort_flag;
    int tile_slabs[kMaxAccStages];
    uint32_t tile_mask;
    int klist[kMaxKernel];
};

template <int kBits, bool kUniform>
__global__ void __launch_bounds__(kThreads, 1) tc_conv_kernel(TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // stage buffers first (1024-byte aligned for the swizzle atoms), control block after
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_b = smem + p.a_stages * p.a_stage_bytes;   // B ring after the A ring
    uint8_t* ctl_base = smem_b + p.b_stages * p.b_stage_bytes;
    SharedControl& ctl = *reinterpret_cast<SharedControl*>(ctl_base);
    int* tile_rows = reinterpret_cast<int*>(ctl_base + sizeof(SharedControl));  // [acc][256]
    int* nbr = tile_rows + p.acc_stages * kTileRows;                            // [256][stride]
    volatile int* abort_flag = &ctl.abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int units_per_offset = p.c_in / 32;

    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl.full_a[s], kProducerThreads);
            mbar_init(&ctl.full_b[s], kProducerThreads);
            mbar_init(&ctl.a_empty[s], 1);
            mbar_init(&ctl.b_empty[s], 1);
        }
        for (int a = 0; a < p.acc_stages; ++a) {
            mbar_init(&ctl.info_full[a], kProducerThreads);
            mbar_init(&ctl.acc_full[a], 1);
            mbar_init(&ctl.acc_empty[a], kEpilogueThreads);
        }
        ctl.abort_flag = 0;
        ctl.tile_mask = 0;
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

    const int n_out = min(max(__ldg(p.counts + 1), 0), p.out_capacity);
    const int edge_total = min(max(__ldg(p.counts), 0), p.edge_capacity);

    if (warp < 8) {
        // ======================= producers =======================
        // Once a wait gives up (ok == false) a producer keeps walking the tile loop so
        // that the three named-barrier syncs per tile stay matched, but does no work.
        // the stage an A gather overwrites was read two MMAs before the one just released
        const int ahead_a = p.a_stages - 2;
        Ring ring_a{0, 0u}, ring_b{0, 0u};   // persist across tiles
        bool ok = true;
        int local_tile = 0;
        // B chunks this thread fills in every slab: idx = tid + 256 i over [chunk][c_out]
        const int tasks = (p.c_out * 8 + kProducerThreads - 1) / kProducerThreads;
        int task_co[kMaxTasks];
        int task_chunk[kMaxTasks];
#pragma unroll
        for (int i = 0; i < kMaxTasks; ++i) {
            int idx = tid + kProducerThreads * i;
            task_co[i] = idx % p.c_out;
            task_chunk[i] = idx / p.c_out;  // >= 8 means no task
        }
        // per-thread constants of the A gather: rows tid/8 + 32 j, chunk tid % 8
        const int a_chunk = tid & 7;
        const int a_half = a_chunk >> 2;
        uint32_t a_dst[8];
        int a_nbr[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r = (tid >> 3) + 32 * j;
            a_dst[j] = static_cast<uint32_t>(r * 128 + ((a_chunk ^ (r & 7)) << 4));
            a_nbr[j] = r * p.nbr_stride;
        }
        // per-task constants of the B fill
        uint32_t b_dst[kMaxTasks];
        int b_src[kMaxTasks];   // (chunk & 3) * words-per-chunk * c_out + co
#pragma unroll
        for (int i = 0; i < kMaxTasks; ++i) {
            b_dst[i] = static_cast<uint32_t>(task_co[i] * 128 + (((task_chunk[i] & 7) ^ (task_co[i] & 7)) << 4));
            b_src[i] = (task_chunk[i] & 3) * (kBits == 8 ? 2 : 1) * p.c_out + task_co[i];
        }
        const int group_shift = p.group_size >= 128 ? 7 : (p.group_size >= 64 ? 6 : 5);
        // Packed codes of one slab for this thread's B chunks. With kUniform (C_out
        // divides 256) every chunk of a thread has the same output channel, so two
        // (scale | bias << 16) words -- one per slab half -- suffice.
        uint32_t nw0[kMaxTasks], nw1[kMaxTasks], nsb[2], nsbt[kUniform ? 1 : kMaxTasks];
        int cur_units = 0;
        auto load_b = [&](UnitCursor cursor) {
            const uint32_t* wb[2];
            const __half* sp[2];
            const __half* bp[2];
            bool uv[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                uv[u] = cursor.unit < cur_units;
                const int k = uv[u] ? ctl.klist[cursor.offset] : 0;
                const int ci0 = uv[u] ? cursor.slice * 32 : 0;
                const size_t q = (static_cast<size_t>(k) * p.groups + (ci0 >> group_shift)) * p.c_out;
                sp[u] = p.scales + q;
                bp[u] = p.qbiases + q;
                wb[u] = p.packed + (static_cast<size_t>(k) * p.words +
                                    (kBits == 4 ? (ci0 >> 3) : (ci0 >> 2))) * p.c_out;
                cursor.advance(1, units_per_offset);
            }
            if (kUniform) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    nsb[u] = 0u;
                    if (uv[u]) {
                        nsb[u] = ldg_u16_pinned(sp[u] + task_co[0]) |
                                 (ldg_u16_pinned(bp[u] + task_co[0]) << 16);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kMaxTasks; ++i) {
                nw0[i] = 0u;
                nw1[i] = 0u;
                if (!kUniform) {
                    nsbt[i] = 0u;
                }
                if (i < tasks && task_chunk[i] < 8) {
                    const bool second = (task_chunk[i] & 4) != 0;
                    if (second ? uv[1] : uv[0]) {
                        const uint32_t* base = second ? wb[1] : wb[0];
                        nw0[i] = ldg_u32_pinned(base + b_src[i]);
                        if (kBits == 8) {
                            nw1[i] = ldg_u32_pinned(base + b_src[i] + p.c_out);
                        }
                        if (!kUniform) {
                            nsbt[i] = ldg_u16_pinned((second ? sp[1] : sp[0]) + task_co[i]) |
                                      (ldg_u16_pinned((second ? bp[1] : bp[0]) + task_co[i]) << 16);
                        }
                    }
                }
            }
        };
        for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++local_tile) {
            const int a = local_tile % p.acc_stages;
            const uint32_t acc_parity = ((local_tile / p.acc_stages) & 1) ^ 1;
            producer_sync();  // everyone is done with the previous tile's tables
            if (ok) {
                // every slab of the earlier tiles is already published, so this cannot
                // wait on work that only this thread could release
                ok = mbar_wait(&ctl.acc_empty[a], acc_parity, abort_flag, p.status);
            }
            if (!ok) {
                producer_sync();
                producer_sync();
                continue;
            }
            // ---- neighbour table of this tile: one row per producer thread ----
            int position = tile * kTileRows + tid;
            int row = -1;
            if (position < p.out_capacity) {
                row = p.row_order != nullptr ? __ldg(p.row_order + position) : position;
                if (row < 0 || row >= p.out_capacity) {
                    raise_status(p.status, LAT_STATUS_BAD_INDEX);
                    row = -1;
                }
            }
            tile_rows[a * kTileRows + tid] = row;
            int* my_nbr = nbr + tid * p.nbr_stride;
            for (int k = 0; k < p.n_kernels; ++k) {
                my_nbr[k] = -1;
            }
            uint32_t mask = 0;
            if (row >= 0 && row < n_out) {
                int begin = __ldg(p.row_offsets + row);
                int end = __ldg(p.row_offsets + row + 1);
                for (int e = begin; e < end; ++e) {
                    if (e < 0 || e >= edge_total) {
                        continue;
                    }
                    int in_row = __ldg(p.in_rows + e);
                    int k = __ldg(p.kernel_ids + e);
                    if (in_row < 0 || k < 0) {
                        continue;
                    }
                    if (in_row >= p.in_capacity || k >= p.n_kernels) {
                        raise_status(p.status, LAT_STATUS_BAD_INDEX);
                        continue;
                    }
                    my_nbr[k] = in_row;
                    mask |= 1u << k;
                }
            }
            mask = __reduce_or_sync(0xffffffffu, mask);
            if (lane == 0 && mask != 0) {
                atomicOr(&ctl.tile_mask, mask);
            }
            producer_sync();
            const uint32_t tile_mask = ctl.tile_mask;
            if (tid < kMaxKernel) {
                ctl.klist[tid] = static_cast<int>(__fns(tile_mask, 0, tid + 1));
            }
            const int units = __popc(tile_mask) * units_per_offset;
            const int slabs = (units + 1) >> 1;
            if (tid == 0) {
                ctl.tile_slabs[a] = slabs;
            }
            producer_sync();
            if (tid == 0) {
                ctl.tile_mask = 0;  // for the next tile (ordered by the sync at its top)
            }
            mbar_arrive(&ctl.info_full[a]);
            cur_units = units;
            UnitCursor cur_a{a_half, 0, a_half};     // this thread's half of the A slab to gather
            cur_a.advance(0, units_per_offset);
            UnitCursor cur_q{0, 0, 0};               // quantized B: first unit of the slab
            if (kBits != 0 && kUniform && slabs > 0) {
                load_b(cur_q);
                cur_q.advance(2, units_per_offset);
            }

            // ---- slabs ----
            // A rows are gathered `ahead_a` slabs before their MMA (the gather latency is
            // the long one); fp16 B tiles are copied `ahead_b` slabs ahead, quantized B
            // tiles are converted in the step of their own slab from codes that were
            // loaded into registers one step earlier. One cp.async group per step.
            if (kBits == 0) {
                // fp16 weights: A rows and the B tile of a slab share one stage; the copies
                // are asynchronous and signal the stage's barrier themselves when they
                // land, so this loop only blocks on free stages.
                for (int s = 0; s < slabs && ok; ++s) {
                    if (!mbar_wait(&ctl.a_empty[ring_a.index], ring_a.phase ^ 1u, abort_flag,
                                   p.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_addr = smem_u32(smem + ring_a.index * p.a_stage_bytes);
                    const uint32_t b_addr = a_addr + kSlabBytesA;
                    const bool uv = cur_a.unit < units;
                    const int uk = uv ? ctl.klist[cur_a.offset] : 0;
                    const int col = (uv ? cur_a.slice : 0) * 32 + (a_chunk & 3) * 8;
                    cur_a.advance(2, units_per_offset);
                    const __half* col_base = p.feats + col;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int in_row = uv ? nbr[a_nbr[j] + uk] : -1;
                        const bool valid = in_row >= 0;
                        const __half* src =
                            valid ? col_base + static_cast<size_t>(in_row) * p.feat_stride : p.feats;
                        cp_async_16(a_addr + a_dst[j], src, valid);
                    }
                    const __half* base = p.weights + static_cast<size_t>(uk) * p.w_stride_k + col;
                    for (int co = tid >> 3; co < p.c_out; co += 32) {
                        cp_async_16(b_addr + co * 128 + ((a_chunk ^ (co & 7)) << 4),
                                    base + static_cast<size_t>(co) * p.w_stride_co, uv);
                    }
                    cp_async_arrive_noinc(&ctl.full_a[ring_a.index]);
                    ring_a.advance(p.a_stages);
                }
            } else {
                // packed weights: the A gather runs `ahead_a` slabs ahead of the B
                // conversion, each on its own ring
                for (int s = -ahead_a; s < slabs && ok; ++s) {
                    const int sa = s + ahead_a;
                    if (sa < slabs) {
                        if (!mbar_wait(&ctl.a_empty[ring_a.index], ring_a.phase ^ 1u, abort_flag,
                                       p.status)) {
                            ok = false;
                            break;
                        }
                        const uint32_t a_addr = smem_u32(smem + ring_a.index * p.a_stage_bytes);
                        const bool uv = cur_a.unit < units;
                        const int uk = uv ? ctl.klist[cur_a.offset] : 0;
                        const __half* col_base =
                            p.feats + (uv ? cur_a.slice : 0) * 32 + (a_chunk & 3) * 8;
                        cur_a.advance(2, units_per_offset);
                        {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int in_row = uv ? nbr[a_nbr[j] + uk] : -1;
                                const bool valid = in_row >= 0;
                                const __half* src = valid ? col_base + static_cast<size_t>(in_row) *
                                                                           p.feat_stride
                                                          : p.feats;
                                cp_async_16(a_addr + a_dst[j], src, valid);
                            }
                        }
                        cp_async_arrive_noinc(&ctl.full_a[ring_a.index]);
                        ring_a.advance(p.a_stages);
                    }
                    if (s < 0) {
                        continue;
                    }
                    if (!mbar_wait(&ctl.b_empty[ring_b.index], ring_b.phase ^ 1u, abort_flag,
                                   p.status)) {
                        ok = false;
                        break;
                    }
                    uint8_t* stage_b = smem_b + ring_b.index * p.b_stage_bytes;
                    if (!kUniform) {
                        load_b(cur_q);
                        cur_q.advance(2, units_per_offset);
                    }
                    {
                        uint32_t c0[kMaxTasks], c1[kMaxTasks], csb[kUniform ? 2 : kMaxTasks];
#pragma unroll
                        for (int i = 0; i < kMaxTasks; ++i) {
                            c0[i] = nw0[i];
                            c1[i] = nw1[i];
                            if (!kUniform) {
                                csb[i] = nsbt[i];
                            }
                        }
                        if (kUniform) {
                            csb[0] = nsb[0];
                            csb[1] = nsb[1];
                            if (s + 1 < slabs) {
                                load_b(cur_q);  // in flight while this slab is converted
                                cur_q.advance(2, units_per_offset);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < kMaxTasks; ++i) {
                            if (i < tasks && task_chunk[i] < 8) {
                                const uint32_t sb = kUniform ? ((task_chunk[i] & 4) ? csb[1] : csb[0])
                                                             : csb[kUniform ? 0 : i];
                                const __half2 scale = __half2half2(__ushort_as_half(sb & 0xFFFFu));
                                const __half2 qbias = __half2half2(__ushort_as_half(sb >> 16));
                                uint4 value;
                                if (kBits == 4) {
                                    value = dequant_int4(c0[i], scale, qbias);
                                } else {
                                    uint2 lo = dequant_int8(c0[i], scale, qbias);
                                    uint2 hi = dequant_int8(c1[i], scale, qbias);
                                    value = make_uint4(lo.x, lo.y, hi.x, hi.y);
                                }
                                *reinterpret_cast<uint4*>(stage_b + b_dst[i]) = value;
                            }
                        }
                    }
                    fence_proxy_async();  // generic-proxy stores -> visible to the MMA
                    mbar_arrive(&ctl.full_b[ring_b.index]);
                    ring_b.advance(p.b_stages);
                }
            }
        }
        cp_async_wait<0>();
    } else if (warp < 16) {
        // ======================= epilogue =======================
        const int ew = warp - 8;
        const int quarter = ew & 3;       // TMEM lanes 32*quarter .. +31 (warp index % 4)
        const int half_tile = ew >> 2;    // which 128-row half of the tile
        const int tile_row = half_tile * 128 + quarter * 32 + lane;
        bool ok = true;
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int a = local_tile % p.acc_stages;
            const uint32_t parity = (local_tile / p.acc_stages) & 1;
            if (!mbar_wait(&ctl.info_full[a], parity, abort_flag, p.status) ||
                !mbar_wait(&ctl.acc_full[a], parity, abort_flag, p.status)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int slabs = ctl.tile_slabs[a];
            const int row = tile_rows[a * kTileRows + tile_row];
            __half* out_row = row >= 0 ? p.out + static_cast<size_t>(row) * p.c_out : nullptr;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>((2 * a + half_tile) * p.acc_cols);
            for (int c0 = 0; c0 < p.c_out; c0 += 32) {
                uint32_t v[32];
                const int width = min(32, p.c_out - c0);  // 32 or 16
                if (slabs > 0) {
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
            tc_fence_before();
            mbar_arrive(&ctl.acc_empty[a]);
        }
    } else if (lane == 0) {
        // ======================= MMA issuer =======================
        const uint32_t idesc = make_instr_desc(128, p.c_out);
        bool ok = true;
        Ring ring_a{0, 0u}, ring_b{0, 0u};
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int a = local_tile % p.acc_stages;
            const uint32_t parity = (local_tile / p.acc_stages) & 1;
            if (!mbar_wait(&ctl.info_full[a], parity, abort_flag, p.status) ||
                !mbar_wait(&ctl.acc_empty[a], parity ^ 1, abort_flag, p.status)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int slabs = ctl.tile_slabs[a];
            const uint32_t tmem_d0 = tmem_base + static_cast<uint32_t>(2 * a * p.acc_cols);
            const uint32_t tmem_d1 = tmem_d0 + static_cast<uint32_t>(p.acc_cols);
            for (int s = 0; s < slabs; ++s) {
                if (!mbar_wait(&ctl.full_a[ring_a.index], ring_a.phase, abort_flag, p.status) ||
                    (kBits != 0 &&
                     !mbar_wait(&ctl.full_b[ring_b.index], ring_b.phase, abort_flag, p.status))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const int stage_a = ring_a.index;
                const int stage_b = ring_b.index;
                ring_a.advance(p.a_stages);
                ring_b.advance(p.b_stages);
                const uint32_t a_addr = smem_u32(smem + stage_a * p.a_stage_bytes);
                const uint64_t desc_a0 = make_smem_desc(a_addr);
                const uint64_t desc_a1 = make_smem_desc(a_addr + 128 * 128);
                const uint64_t desc_b = make_smem_desc(
                    kBits == 0 ? a_addr + kSlabBytesA : smem_u32(smem_b + stage_b * p.b_stage_bytes));
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    // 16 fp16 = 32 bytes along K inside the swizzle atom: +2 in 16-byte units
                    const uint32_t acc = (s | kk) != 0 ? 1u : 0u;
                    umma_f16(tmem_d0, desc_a0 + 2 * kk, desc_b + 2 * kk, idesc, acc);
                    umma_f16(tmem_d1, desc_a1 + 2 * kk, desc_b + 2 * kk, idesc, acc);
                }
                umma_commit(&ctl.a_empty[stage_a]);
                if (kBits != 0) {
                    umma_commit(&ctl.b_empty[stage_b]);
                }
            }
            if (!ok) {
                break;
            }
            if (slabs > 0) {
                umma_commit(&ctl.acc_full[a]);
            } else {
                mbar_arrive(&ctl.acc_full[a]);
            }
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

// fp16 (K, C_in, C_out) -> (K, C_out, C_in) so that B rows are K-major
__global__ void transpose_weights_kernel(const __half* in, int K, int c_in, int c_out, __half* out) {
    size_t total = static_cast<size_t>(K) * c_in * c_out;
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (i >= total) {
        return;
    }
    int ci = static_cast<int>(i % c_in);
    size_t rest = i / c_in;
    int co = static_cast<int>(rest % c_out);
    int k = static_cast<int>(rest / c_out);
    out[i] = in[(static_cast<size_t>(k) * c_in + ci) * c_out + co];
}

// packed int4/int8 (K, S*bits/32, C_out) + scales/biases (K, S/group, C_out) ->
// fp16 (K, C_out, C_in) = code*scale + bias evaluated in float32 and rounded once
__global__ void stage_quantized_weights_kernel(
    const uint32_t* packed, const __half* scales, const __half* biases, int K, int c_in, int c_out,
    int words, int groups, int group_size, int bits, __half* out
) {
    size_t total = static_cast<size_t>(K) * c_in * c_out;
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (i >= total) {
        return;
    }
    // consecutive threads -> consecutive co (coalesced reads); writes are strided
    int co = static_cast<int>(i % c_out);
    size_t rest = i / c_out;
    int ci = static_cast<int>(rest % c_in);
    int k = static_cast<int>(rest / c_in);
    int bit = ci * bits;
    uint32_t word = __ldg(packed + (static_cast<size_t>(k) * words + (bit >> 5)) * c_out + co);
    uint32_t code = (word >> (bit & 31)) & ((1u << bits) - 1u);
    size_t q = (static_cast<size_t>(k) * groups + ci / group_size) * c_out + co;
    float w = fmaf(static_cast<float>(code), __half2float(__ldg(scales + q)),
                   __half2float(__ldg(biases + q)));
    out[(static_cast<size_t>(k) * c_out + co) * c_in + ci] = __float2half_rn(w);
}

int pow2_at_least(int value, int floor_value) {
    int out = floor_value;
    while (out < value) {
        out <<= 1;
    }
    return out;
}

} // namespace

// conv_tc_plan.cu
int run_tc_conv_plan(
    const void* feats, int in_channels, long long feat_stride, const void* feats2, int split,
    long long feat2_stride, const void* weights,
    long long w_stride_k, long long w_stride_co, int n_kernels, int out_channels, int out_capacity,
    const void* bias, const int32_t* row_order, const void* plan, void* out, int32_t* status,
    cudaStream_t stream);

// Packed weights reach the B tiles either converted in registers inside the kernel or
// staged once per call as fp16 (default; LAT_TC_DEQUANT=register selects the former).
static bool dequant_in_registers() {
    const char* mode = std::getenv("LAT_TC_DEQUANT");
    return mode != nullptr && mode[0] == 'r';
}

int run_stage_quantized_weights(
    const uint32_t* packed, const void* scales, const void* biases, int n_kernels, int in_channels,
    int out_channels, int storage_in_channels, int group_size, int bits, void* out, cudaStream_t stream
) {
    const size_t total = static_cast<size_t>(n_kernels) * in_channels * out_channels;
    if (total == 0) {
        return LAT_OK;
    }
    stage_quantized_weights_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(
        packed, static_cast<const __half*>(scales), static_cast<const __half*>(biases), n_kernels,
        in_channels, out_channels, storage_in_channels * bits / 32, storage_in_channels / group_size,
        group_size, bits, static_cast<__half*>(out));
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

bool tc_conv_supported(int dtype, int n_kernels, int in_channels, int out_channels,
                       int quantized_bits, int group_size) {
    if (dtype != LAT_F16) {
        return false;
    }
    if (n_kernels < 1 || n_kernels > kMaxKernel) {
        return false;
    }
    if (in_channels % 32 != 0 || in_channels < 32) {
        return false;
    }
    if (out_channels % 16 != 0 || out_channels < 16 || out_channels > 256) {
        return false;
    }
    if (quantized_bits != 0) {
        if (quantized_bits != 4 && quantized_bits != 8) {
            return false;
        }
        if (group_size % 32 != 0) {
            return false;
        }
    }
    return true;
}

size_t tc_conv_workspace_bytes(int n_kernels, int in_channels, int out_channels) {
    return align_up(sizeof(__half) * static_cast<size_t>(std::max(n_kernels, 1)) *
                    std::max(in_channels, 1) * std::max(out_channels, 1));
}

int run_tc_conv(
    const void* feats, int in_capacity, int in_channels, long long feat_stride,
    const void* feats2, int feats2_channels, long long feat2_stride,
    const void* weights, int weight_layout, const uint32_t* packed, const void* scales,
    const void* biases, int storage_in_channels, int group_size, int bits, int out_channels,
    const int32_t* in_rows, const int32_t* kernel_ids, int edge_capacity, const int32_t* counts,
    const int32_t* row_offsets, int out_capacity, int n_kernels, const void* bias,
    const int32_t* row_order, const void* plan, void* out, void* workspace,
    size_t workspace_bytes, int32_t* status, cudaStream_t stream
) {
    if (out_capacity == 0) {
        return LAT_OK;
    }
    LAT_REQUIRE(feat_stride % 8 == 0 && reinterpret_cast<uintptr_t>(feats) % 16 == 0,
                "feature rows must be 16-byte aligned for the tensor-core route.");
    TcParams p{};
    p.feats = static_cast<const __half*>(feats);
    p.feat_stride = feat_stride;
    p.in_capacity = in_capacity;
    p.c_in = in_channels;
    p.c_out = out_channels;
    p.n_kernels = n_kernels;
    if (packed == nullptr) {
        if (weight_layout == LAT_WEIGHT_OUT_MAJOR) {
            // (K, C_out, C_in): the form lat_dequantize_conv_weights writes
            p.weights = static_cast<const __half*>(weights);
            p.w_stride_k = static_cast<long long>(out_channels) * in_channels;
            p.w_stride_co = in_channels;
        } else if (weight_layout == LAT_WEIGHT_DENSE_5D) {
            // (C_out, K, C_in): rows already K-major
            p.weights = static_cast<const __half*>(weights);
            p.w_stride_k = in_channels;
            p.w_stride_co = static_cast<long long>(n_kernels) * in_channels;
        } else {
            Workspace ws(workspace, workspace_bytes);
            size_t total = static_cast<size_t>(n_kernels) * in_channels * out_channels;
            __half* wt = ws.take<__half>(total);
            if (!ws.ok) {
                return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the convolution.");
            }
            transpose_weights_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(
                static_cast<const __half*>(weights), n_kernels, in_channels, out_channels, wt);
            LAT_LAUNCH_CHECK();
            p.weights = wt;
            p.w_stride_k = static_cast<long long>(out_channels) * in_channels;
            p.w_stride_co = in_channels;
        }
    } else if (!dequant_in_registers()) {
        // staged route: the whole weight is dequantised to fp16 once per call (a few MB,
        // L2-resident) and the B tiles are then plain asynchronous copies
        Workspace ws(workspace, workspace_bytes);
        size_t total = static_cast<size_t>(n_kernels) * in_channels * out_channels;
        __half* wt = ws.take<__half>(total);
        if (!ws.ok) {
            return fail(LAT_WORKSPACE_TOO_SMALL, "workspace is too small for the convolution.");
        }
        stage_quantized_weights_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, stream>>>(
            packed, static_cast<const __half*>(scales), static_cast<const __half*>(biases),
            n_kernels, in_channels, out_channels, storage_in_channels * bits / 32,
            storage_in_channels / group_size, group_size, bits, wt);
        LAT_LAUNCH_CHECK();
        p.weights = wt;
        p.w_stride_k = static_cast<long long>(out_channels) * in_channels;
        p.w_stride_co = in_channels;
        packed = nullptr;
        bits = 0;
    } else {
        p.packed = packed;
        p.scales = static_cast<const __half*>(scales);
        p.qbiases = static_cast<const __half*>(biases);
        p.words = storage_in_channels * bits / 32;
        p.groups = storage_in_channels / group_size;
        p.group_size = group_size;
    }
    if (plan != nullptr && packed == nullptr) {
        // fp16 weights and a prebuilt gather plan: the plan-driven kernel
        return run_tc_conv_plan(feats, in_channels, feat_stride, feats2, in_channels - feats2_channels,
                                feat2_stride, p.weights, p.w_stride_k,
                                p.w_stride_co, n_kernels, out_channels, out_capacity, bias, row_order, plan,
                                out, status, stream);
    }
    LAT_REQUIRE(feats2 == nullptr, "a second feature source needs a gather plan (lat_build_conv_plan).");
    p.in_rows = in_rows;
    p.kernel_ids = kernel_ids;
    p.row_offsets = row_offsets;
    p.counts = counts;
    p.edge_capacity = edge_capacity;
    p.out_capacity = out_capacity;
    p.bias = static_cast<const __half*>(bias);
    p.row_order = row_order;
    p.out = static_cast<__half*>(out);
    p.status = status;
    p.b_stage_bytes = out_channels * 128;
    p.acc_cols = pow2_at_least(out_channels, 32);
    p.acc_stages = std::min(kMaxAccStages, 512 / (2 * p.acc_cols));
    p.tmem_cols = p.acc_stages * 2 * p.acc_cols;
    p.nbr_stride = n_kernels | 1;
    p.ctl_bytes = static_cast<int>(align_up(
        sizeof(SharedControl) + sizeof(int) * kTileRows * (p.acc_stages + p.nbr_stride), 16));
    // keep every B stage on a 1024-byte boundary (the swizzle pattern repeats every
    // eight 128-byte rows)
    p.b_stage_bytes = static_cast<int>(align_up(p.b_stage_bytes, 1024));
    const int smem_budget = 227 * 1024 - 1024 /*alignment slack*/ - p.ctl_bytes;
    if (packed == nullptr) {
        // fp16 weights: one ring, a stage holds the A rows and the B tile
        p.a_stage_bytes = kSlabBytesA + p.b_stage_bytes;
        p.b_stages = 0;
        p.a_stages = std::min(kMaxStages, smem_budget / p.a_stage_bytes);
    } else {
        p.a_stage_bytes = kSlabBytesA;
        p.b_stages = 2;
        p.a_stages = std::min(kMaxStages, (smem_budget - p.b_stages * p.b_stage_bytes) / kSlabBytesA);
    }
    LAT_REQUIRE(p.a_stages >= 2, "internal: shared-memory plan leaves no room for the stage ring.");
    p.num_tiles = (out_capacity + kTileRows - 1) / kTileRows;
    size_t smem_bytes = 1024 + static_cast<size_t>(p.a_stages) * p.a_stage_bytes +
                        static_cast<size_t>(p.b_stages) * p.b_stage_bytes + p.ctl_bytes;
    LAT_REQUIRE(smem_bytes <= 227 * 1024, "internal: shared-memory plan exceeds the SM.");

    int device = 0;
    LAT_CUDA_CHECK(cudaGetDevice(&device));
    int sm_count = 0;
    LAT_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    int grid = std::max(1, std::min(p.num_tiles, sm_count));
    const bool uniform = bits != 0 && kProducerThreads % out_channels == 0;
    auto kernel = bits == 4 ? (uniform ? tc_conv_kernel<4, true> : tc_conv_kernel<4, false>)
                : bits == 8 ? (uniform ? tc_conv_kernel<8, true> : tc_conv_kernel<8, false>)
                            : tc_conv_kernel<0, false>;
    LAT_CUDA_CHECK(cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)));
    kernel<<<grid, kThreads, smem_bytes, stream>>>(p);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // namespace lat

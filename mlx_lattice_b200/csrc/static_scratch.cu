// lat_lookup_coords_static: first-row lookup of query coordinates that allocates
// nothing, for callers that are not allowed to.
//
// Some hosts hand a library a fixed set of device buffers at start-up and forbid any
// later allocation: a control loop with a hard latency budget (an allocation may
// synchronise the device or fail at the worst moment), a process whose device memory
// is fully budgeted by its owner, code that runs after the framework around it has
// frozen its allocator. The regular lat_lookup_coords needs a caller-provided
// workspace for its hash table; such callers may have no spare buffer to give. This
// variant keeps the table in a file-scope __device__ array of fixed size instead.
//
// Consequences of that choice, all part of the contract:
//  - every GPU that loads the library carries the array (2 MiB) until the process exits;
//  - at most kStaticLookupMaxRows source rows; larger inputs are rejected;
//  - the array is shared by every call and keeps the previous call's contents, so each
//    call clears the part it uses first, and two calls that overlap on the GPU (different
//    streams, or different host threads) race on it -- serialise them;
//  - the first call on a device resolves the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it; make that first
//    call outside any stream capture.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace lat {

namespace {

constexpr int kStaticLookupMaxRows = 1 << 18;                 // 262,144 source rows
constexpr int kStaticTableSlots = 2 * kStaticLookupMaxRows;   // 2 MiB of int32 slots
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the symbol, not a device address: the
// kernels below get the address that cudaGetSymbolAddress returns.
static __device__ __align__(256) int32_t g_static_lookup_table[kStaticTableSlots];

std::mutex g_setup_mutex;
int32_t* g_table_address[kMaxDevices] = {};

// Device address of the table on the current device, resolved once per device.
int static_table(int32_t** out) {
    int device = 0;
    LAT_CUDA_CHECK(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) {
        return fail(LAT_INVALID_ARGUMENT, "device index is outside the supported range.");
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_table_address[device] == nullptr) {
        void* address = nullptr;
        LAT_CUDA_CHECK(cudaGetSymbolAddress(&address, g_static_lookup_table));
        g_table_address[device] = static_cast<int32_t*>(address);
    }
    *out = g_table_address[device];
    return LAT_OK;
}

__global__ void static_insert_kernel(
    const int32_t* coords, int rows, int32_t* table, uint32_t mask, int32_t* status
) {
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) {
        return;
    }
    PlainKey key_of{coords};
    if (!table32_insert(table, mask, row, key_of(row), key_of, nullptr)) {
        raise_status(status, LAT_STATUS_HASH_FULL);
    }
}

__global__ void static_lookup_kernel(
    const int32_t* coords, const int32_t* table, uint32_t mask, const int32_t* queries,
    int query_rows, int32_t* out_rows
) {
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row < query_rows) {
        out_rows[row] = table32_find(table, mask, load_coord(queries, row), PlainKey{coords});
    }
}

} // namespace

} // namespace lat

using namespace lat;

extern "C" {

int32_t lat_lookup_coords_static_max_rows(void) { return kStaticLookupMaxRows; }

int lat_lookup_coords_static(
    const int32_t* coords, int32_t rows, const int32_t* queries, int32_t query_rows,
    int32_t* out_rows, int32_t* status, void* stream_ptr
) {
    LAT_REQUIRE(rows >= 0 && query_rows >= 0, "coords must have shape (N, 4).");
    LAT_REQUIRE(rows <= kStaticLookupMaxRows,
                "lat_lookup_coords_static holds at most 262144 source rows in its built-in "
                "table; use lat_lookup_coords with a workspace for larger inputs.");
    LAT_REQUIRE((coords != nullptr || rows == 0) && (queries != nullptr || query_rows == 0) &&
                    (out_rows != nullptr || query_rows == 0),
                "coords, queries and out_rows are required.");
    if (query_rows == 0) {
        return LAT_OK;
    }
    cudaStream_t stream = as_stream(stream_ptr);
    int32_t* table = nullptr;
    int rc = static_table(&table);
    if (rc != LAT_OK) {
        return rc;
    }
    // only the slots this call can touch are cleared (the rest may hold stale rows of an
    // earlier, larger call, but the slot mask keeps them out of reach)
    int capacity = next_pow2(std::max(2LL * rows, 1LL));
    uint32_t mask = static_cast<uint32_t>(capacity - 1);
    LAT_CUDA_CHECK(cudaMemsetAsync(table, 0xFF, sizeof(int32_t) * capacity, stream));
    if (rows > 0) {
        static_insert_kernel<<<(rows + 255) / 256, 256, 0, stream>>>(coords, rows, table, mask, status);
        LAT_LAUNCH_CHECK();
    }
    static_lookup_kernel<<<(query_rows + 255) / 256, 256, 0, stream>>>(
        coords, table, mask, queries, query_rows, out_rows);
    LAT_LAUNCH_CHECK();
    return LAT_OK;
}

} // extern "C"

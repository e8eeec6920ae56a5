// An entry point for callers that must not allocate device memory.
//
// Who that is: a serving process that hands all of the GPU's memory to its own
// pool at start-up (any later cudaMalloc fails or eats into the pool's head
// room), and latency-sensitive threads for which cudaMalloc / cudaFree are off
// limits because they synchronise the whole device and stall every other
// stream while they run.  Such a caller cannot create a stage object (which
// allocates its working buffers once) nor ask torch for temporaries; it owns
// its inputs and outputs and nothing else.
//
// pa_search_reduced_noalloc runs entry routing followed by the traversal --
// the same two kernels pa_route and pa_traverse_packed launch -- and keeps the
// intermediate entry tables (ids and distances, [batch, n_leaves]) in a
// file-scope device array instead of caller- or library-allocated memory.
// The array is part of the library image: every GPU that loads the library
// holds PA_NOALLOC_SCRATCH_BYTES of it until the process exits.
#include <mutex>

#include "pa_common.cuh"

namespace pa {

constexpr size_t kEntryElems =
    static_cast<size_t>(PA_NOALLOC_MAX_BATCH) * PA_NOALLOC_MAX_LEAVES;

// In HOST code this name is only a stand-in for the symbol, not a device
// address; the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_entry_scratch[PA_NOALLOC_SCRATCH_BYTES];
static_assert(PA_NOALLOC_SCRATCH_BYTES == kEntryElems * (sizeof(int64_t) + sizeof(float)),
              "scratch size and its layout disagree");

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static void *g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device.  The first call
// on a device performs the symbol lookup (which may initialise the context and
// load the module), so it should happen before any stream capture begins.
static int scratch_on_current_device(unsigned char **out) {
    int dev = -1;
    PA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices)
        return fail(PA_ERR_ARG, "device ordinal %d outside [0, %d)", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void *addr = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&addr, g_entry_scratch);
        if (err != cudaSuccess) return cuda_fail(err, "cudaGetSymbolAddress(g_entry_scratch)");
        if (addr == nullptr) return fail(PA_ERR_CUDA, "scratch symbol resolved to a null address");
        g_scratch_addr[dev] = addr;
    }
    *out = static_cast<unsigned char *>(g_scratch_addr[dev]);
    return PA_OK;
}

}  // namespace pa

extern "C" int pa_search_reduced_noalloc(
    int64_t *output_I, float *output_D, const int32_t *packed_nbr, const int32_t *row_of,
    const float *storage, const float *query, const float *route_vectors,
    const int64_t *entry_nodes, const float *entry_vectors, int64_t batch, int64_t n_nodes,
    int64_t n_storage, int d_principle, int n_neighbors, int n_routers, int n_leaves,
    int ef_search, void *stream_) {
    using namespace pa;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PA_REQUIRE(batch >= 0, "batch must not be negative");
    if (batch > PA_NOALLOC_MAX_BATCH)
        return fail(PA_ERR_ARG,
                    "batch %lld exceeds PA_NOALLOC_MAX_BATCH (%d): the static scratch holds "
                    "entry tables for at most that many queries; split the batch",
                    static_cast<long long>(batch), PA_NOALLOC_MAX_BATCH);
    if (n_leaves > PA_NOALLOC_MAX_LEAVES)
        return fail(PA_ERR_ARG, "n_leaves %d exceeds PA_NOALLOC_MAX_LEAVES (%d)", n_leaves,
                    PA_NOALLOC_MAX_LEAVES);
    PA_REQUIRE(n_leaves > 0 && n_leaves % 32 == 0, "n_leaves must be a multiple of 32");
    PA_REQUIRE(route_vectors != nullptr ? n_routers > 0 : true, "n_routers must be positive");
    PA_REQUIRE(d_principle > 0 && d_principle % 4 == 0 && d_principle <= 4096,
               "d_principle must be a multiple of 4 (at most 4096)");
    if (batch == 0) return PA_OK;
    PA_REQUIRE(query && entry_nodes && entry_vectors, "null pointer");
    PA_REQUIRE(aligned16(query) && aligned16(entry_vectors) &&
                   (route_vectors == nullptr || aligned16(route_vectors)),
               "vectors must be 16-byte aligned");
    unsigned char *scratch = nullptr;
    int rc = scratch_on_current_device(&scratch);
    if (rc != PA_OK) return rc;
    // every check of the traversal runs before the routing kernel is enqueued: a
    // refused call launches nothing
    rc = traverse_packed_check(output_I, output_D, packed_nbr, row_of, storage, query, d_principle,
                               reinterpret_cast<const int64_t *>(scratch),
                               reinterpret_cast<const float *>(scratch), batch, n_nodes,
                               d_principle, n_neighbors, n_leaves, ef_search);
    if (rc != PA_OK) return rc;
    // layout: ids for MAX_BATCH x MAX_LEAVES first, distances after them; rows are
    // packed at the call's own n_leaves.  Every element the traversal reads is
    // written by the routing kernel of this same call, so nothing needs clearing.
    int64_t *entry_I = reinterpret_cast<int64_t *>(scratch);
    float *entry_D = reinterpret_cast<float *>(scratch + kEntryElems * sizeof(int64_t));
    rc = route_launch(nullptr, entry_D, entry_I, query, d_principle, route_vectors, entry_nodes,
                      entry_vectors, batch, d_principle, route_vectors ? n_routers : 1, n_leaves,
                      nullptr, nullptr, stream);
    if (rc != PA_OK) return rc;
    return traverse_packed_launch(output_I, output_D, packed_nbr, row_of, storage, query,
                                  d_principle, entry_I, entry_D, batch, n_nodes, n_storage,
                                  d_principle, n_neighbors, n_leaves, ef_search, nullptr, stream);
}

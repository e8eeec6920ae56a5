// Builds the packed device-resident index from upstream's CSR tensors: the
// counterpart of the device copies prepared by IndexStaged.to
// (pilot_ann/layers/staged.py:124-139).  One warp per node.
#include "pa_common.cuh"

namespace pa {

__global__ void pack_fill_kernel(int4 *nbr, int64_t n_slots, int n_nb) {
    int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < n_slots) nbr[i] = make_int4((i % n_nb) == 0 ? kEmptyRowTag : -1, -1, 0, 0);
}

__global__ void pack_rows_kernel(int4 *__restrict__ nbr, int32_t *__restrict__ row_of,
                                 const int64_t *__restrict__ indptr,
                                 const int64_t *__restrict__ indices,
                                 const int64_t *__restrict__ mapping, int64_t n_nodes,
                                 int64_t n_storage, int n_nb, int *__restrict__ error) {
    const int lane = threadIdx.x & 31;
    const int64_t u = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (u >= n_nodes) return;
    const int64_t row = mapping[u];
    const int64_t lo = indptr[u], hi = indptr[u + 1];
    if (lane == 0) row_of[u] = row < 0 ? -1 : static_cast<int32_t>(row);
    if (row >= n_storage || row > 0x7ffffffe) { if (lane == 0) atomicMax(error, 2); return; }
    if (row < 0) {
        // a node without a vector row cannot carry an adjacency row here
        if (hi != lo && lane == 0) atomicMax(error, 1);
        return;
    }
    const int64_t len = min(hi - lo, static_cast<int64_t>(n_nb));
    if (len <= 0) return;  // keeps the "empty row" tag written by the fill pass
    for (int i = lane; i < n_nb; i += 32) {
        int2 e = make_int2(-1, -1);
        if (i < len) {
            int64_t v = indices[lo + i];
            if (v >= n_nodes) { atomicMax(error, 2); v = -1; }
            if (v >= 0) {
                // an id that repeats an earlier slot of the row: every search finds it
                // visited by then (the bloom filter of the traversal, the exact marks
                // of the refinement), so the slot is tagged and skipped
                bool dup = false;
                for (int j = 0; j < i; ++j) dup = dup || indices[lo + j] == v;
                int64_t r = mapping[v];
                e = dup ? make_int2(kDupTag, -1)
                        : make_int2(static_cast<int32_t>(v), r < 0 ? -1 : static_cast<int32_t>(r));
            }
        }
        // the bloom probes of the slot: a chunk of 32 slots is what the search
        // tests-and-sets together, so the elections are a property of the row
        const uint2 probe = probe_pack(bloom_prepare(e.x, lane));
        nbr[row * n_nb + i] = make_int4(e.x, e.y, static_cast<int>(probe.x),
                                        static_cast<int>(probe.y));
    }
}

}  // namespace pa

extern "C" int pa_pack_graph(int32_t *packed_nbr, int32_t *row_of, const int64_t *indptr,
                             const int64_t *indices, const int64_t *mapping, int64_t n_nodes,
                             int64_t n_storage, int n_neighbors, void *stream_) {
    using namespace pa;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PA_REQUIRE(n_neighbors > 0 && n_neighbors % 32 == 0, "n_neighbors must be a multiple of 32");
    PA_REQUIRE(n_nodes >= 0 && n_nodes < 0x7fffffff && n_storage >= 0 && n_storage < 0x7fffffff,
               "ids must fit int32");
    PA_REQUIRE(packed_nbr && row_of && indptr && indices && mapping, "null pointer");
    PA_REQUIRE((reinterpret_cast<uintptr_t>(packed_nbr) & 15u) == 0,
               "packed_nbr must be 16-byte aligned");
    // error word of the row kernel (the more severe code wins); released on every
    // way out of this function
    struct ErrorWord {
        int *p = nullptr;
        cudaStream_t s;
        ~ErrorWord() { if (p != nullptr) cudaFreeAsync(p, s); }
    } word;
    word.s = stream;
    PA_CUDA_TRY(cudaMallocAsync(&word.p, sizeof(int), stream));
    int *error = word.p;
    PA_CUDA_TRY(cudaMemsetAsync(error, 0, sizeof(int), stream));
    const int64_t n_slots = n_storage * n_neighbors;
    if (n_slots > 0) {
        pack_fill_kernel<<<static_cast<unsigned>((n_slots + 255) / 256), 256, 0, stream>>>(
            reinterpret_cast<int4 *>(packed_nbr), n_slots, n_neighbors);
        count_launch();
    }
    if (n_nodes > 0) {
        const int64_t threads = n_nodes * 32;
        pack_rows_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
            reinterpret_cast<int4 *>(packed_nbr), row_of, indptr, indices, mapping, n_nodes,
            n_storage, n_neighbors, error);
        count_launch();
    }
    PA_CUDA_TRY(cudaGetLastError());
    int host_error = 0;
    PA_CUDA_TRY(cudaMemcpyAsync(&host_error, error, sizeof(int), cudaMemcpyDeviceToHost, stream));
    PA_CUDA_TRY(cudaStreamSynchronize(stream));
    if (host_error == 1)
        return fail(PA_ERR_UNPACKABLE, "a node with neighbours has no storage row (mapping < 0)");
    if (host_error == 2) return fail(PA_ERR_UNPACKABLE, "an id or storage row is out of range");
    return PA_OK;
}

// Visited-set pool on the device: the counterpart of upstream's Bitmask /
// BitmaskPool (extension/inc/bitmask.hpp:12-45, 51-76), which hands every CPU
// worker thread an int32-per-node array stamped with an epoch marker so that it
// never has to be cleared between queries.
//
// Here a "worker" is a resident CTA of the refinement kernel.  The pool holds
// n_slots arrays of one byte per node plus the last marker each slot used.  CTA i
// of a launch owns slot (slot_begin + i) for the whole launch -- that is the
// get / put of upstream's pool, decided by the launch geometry instead of a
// mutex-guarded queue -- bumps the slot's marker once per query (1 .. 254) and
// wipes the slot's array when the markers run out, as Bitmask::advance does on
// wrap-around.  A byte equal to the current marker means "visited by this query".
// Memory: n_slots * round_up(n_nodes, 16) bytes, allocated once.  Beside the markers the
// pool keeps one counter per slot: the CTAs of a launch claim the queries beyond their
// first through the counter of the launch's first slot (cleared before the launch).
//
// Launches that may run concurrently (different streams) must use disjoint slot
// ranges; the stage object gives each of its streams its own range.
#include <new>

#include "pa_common.cuh"

struct pa_visited_pool {
    uint8_t *marks = nullptr;
    int32_t *epoch = nullptr;  // [n_slots] last markers, then [n_slots] claim counters
    int64_t n_nodes = 0, slot_stride = 0;
    int n_slots = 0, device = 0;
};

namespace pa {

static int64_t slot_stride_for(int64_t n_nodes) { return (n_nodes + 15) / 16 * 16; }

void pool_view(const pa_visited_pool *pool, uint8_t **marks, int32_t **epoch, int64_t *slot_stride,
               int *n_slots, int64_t *n_nodes) {
    *marks = pool->marks; *epoch = pool->epoch; *slot_stride = pool->slot_stride;
    *n_slots = pool->n_slots; *n_nodes = pool->n_nodes;
}

}  // namespace pa

extern "C" int64_t pa_visited_pool_bytes(int64_t n_nodes, int n_slots) {
    if (n_nodes <= 0 || n_slots <= 0) return 0;
    return pa::slot_stride_for(n_nodes) * n_slots + 2 * static_cast<int64_t>(sizeof(int32_t)) * n_slots;
}

extern "C" int pa_visited_pool_create(pa_visited_pool **out, int64_t n_nodes, int n_slots) {
    using namespace pa;
    PA_REQUIRE(out != nullptr, "null pointer");
    *out = nullptr;
    PA_REQUIRE(n_nodes > 0 && n_nodes < 0x7fffffff, "node ids must fit int32");
    PA_REQUIRE(n_slots > 0 && n_slots <= (1 << 20), "n_slots out of range");
    pa_visited_pool *pool = new (std::nothrow) pa_visited_pool();
    if (pool == nullptr) return fail(PA_ERR_CUDA, "out of host memory");
    pool->n_nodes = n_nodes;
    pool->n_slots = n_slots;
    pool->slot_stride = slot_stride_for(n_nodes);
    cudaError_t e = cudaGetDevice(&pool->device);
    const size_t bytes = static_cast<size_t>(pool->slot_stride) * n_slots;
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&pool->marks), bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&pool->epoch), 2 * sizeof(int32_t) * n_slots);
    if (e == cudaSuccess) e = cudaMemset(pool->marks, 0, bytes);
    if (e == cudaSuccess) e = cudaMemset(pool->epoch, 0, 2 * sizeof(int32_t) * n_slots);
    if (e != cudaSuccess) {
        pa_visited_pool_destroy(pool);
        return cuda_fail(e, "visited pool allocation");
    }
    *out = pool;
    return PA_OK;
}

extern "C" void pa_visited_pool_destroy(pa_visited_pool *pool) {
    if (pool == nullptr) return;
    int previous = -1;
    const bool switched = cudaGetDevice(&previous) == cudaSuccess && previous != pool->device &&
                          cudaSetDevice(pool->device) == cudaSuccess;
    cudaFree(pool->marks);
    cudaFree(pool->epoch);
    if (switched) cudaSetDevice(previous);
    delete pool;
}

extern "C" int pa_visited_pool_slots(const pa_visited_pool *pool) {
    return pool == nullptr ? 0 : pool->n_slots;
}

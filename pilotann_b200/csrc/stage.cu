// The per-device search-stage object: streams, device-side working buffers and
// the chunked copy-in / project / route / traverse / copy-back schedule.
// Replaces the GPU half of upstream `pipeline` (extension/pipeline_cpu.cpp:
// 32-145): its process-global static stream pool (:67-75, bound to whichever
// device was current at the first call), the per-call allocation of device and
// pinned buffers (:78-96) and the launch + asynchronous copy-back per chunk
// (:120-140).  Buffers are allocated once, at creation; a call allocates
// nothing.
#include <new>
#include <vector>

#include "pa_common.cuh"

struct pa_stage {
    pa_stage_index ix;
    int device = 0;
    int64_t max_batch = 0;
    int max_ef = 0;
    std::vector<cudaStream_t> streams;
    cudaStream_t copy_stream = nullptr;     // carries the rotated queries back while a chunk searches
    std::vector<cudaEvent_t> projected;     // per stream: the chunk's rotated queries are ready
    float *d_raw = nullptr;      // [max_batch, d_model] raw queries (copy-in target)
    float *d_rot = nullptr;      // [max_batch, d_model] rotated queries
    int64_t *d_router = nullptr; // [max_batch]
    float *d_ep_D = nullptr;     // [max_batch, n_leaves]
    int64_t *d_ep_I = nullptr;   // [max_batch, n_leaves]
    float *d_dots = nullptr;     // [max_batch, n_routers] tensor-core router scores
    float *d_rnorm = nullptr;    // [n_routers] squared router norms
    int64_t *d_out_I = nullptr;  // [max_batch, 4, max_ef]
    float *d_out_D = nullptr;
    // refinement on the GPU (pa_stage_attach_refine)
    pa_refine_index rx = {};
    bool has_refine = false;
    pa_visited_pool *pool = nullptr;  // slots_per_stream slots for each stream
    int slots_per_stream = 0;
    int64_t *d_ref_I = nullptr;  // [max_batch, 4 * max_ef] stage-2 rows or top-k
    float *d_ref_D = nullptr;
    // persistent pinned buffers of the submit / wait slots (one slot per stream)
    int64_t slot_rows = 0;       // queries a slot can take: max_batch / n_streams
    int64_t *h_slot_I = nullptr; // [n_streams, slot_rows, 4 * max_ef]
    float *h_slot_D = nullptr;
    float *h_slot_rot = nullptr; // [n_streams, slot_rows, d_model]
    std::vector<cudaEvent_t> slot_done;
    std::vector<int64_t> slot_pending;  // rows in flight per slot, -1 = idle
};

namespace pa {

struct DeviceScope {
    int previous = -1;
    bool switched = false;
    cudaError_t enter(int device) {
        cudaError_t e = cudaGetDevice(&previous);
        if (e != cudaSuccess) return e;
        if (previous != device) {
            e = cudaSetDevice(device);
            switched = (e == cudaSuccess);
        }
        return e;
    }
    ~DeviceScope() {
        if (switched) cudaSetDevice(previous);
    }
};

// project (if the index has a rotation) -> route -> traverse for rows
// [0, n) of the given buffers, all on one stream.
static int enqueue_chunk(pa_stage *st, const float *raw, float *rot, int64_t *router,
                         float *dots, float *ep_D, int64_t *ep_I, int64_t *out_I, float *out_D, int64_t n,
                         int ef, int32_t *stats, cudaStream_t stream,
                         cudaEvent_t projected = nullptr) {
    const pa_stage_index &ix = st->ix;
    const float *rotated = raw;
    if (ix.VT != nullptr) {
        int rc = project_launch(rot, raw, ix.VT, n, ix.d_model, ix.d_model, ix.d_model, stream);
        if (rc != PA_OK) return rc;
        rotated = rot;
    }
    if (projected != nullptr) PA_CUDA_TRY(cudaEventRecord(projected, stream));
    int rc = route_launch(router, ep_D, ep_I, rotated, ix.d_model, ix.route_vectors,
                          ix.entry_nodes, ix.entry_vectors, n, ix.d_principle,
                          ix.route_vectors ? ix.n_routers : 1, ix.n_leaves, dots, st->d_rnorm,
                          stream);
    if (rc != PA_OK) return rc;
    return traverse_packed_launch(out_I, out_D, ix.packed_nbr, ix.row_of, ix.storage, rotated,
                                  ix.d_model, ep_I, ep_D, n, ix.n_nodes, ix.n_storage,
                                  ix.d_principle, ix.n_neighbors, ix.n_leaves, ef, stats, stream);
}

static int check_call(pa_stage *st, int64_t batch, int ef) {
    if (st == nullptr) return fail(PA_ERR_STATE, "stage is null");
    PA_REQUIRE(batch >= 0 && batch <= st->max_batch, "batch exceeds the stage's max_batch");
    PA_REQUIRE(ef > 0 && ef <= st->max_ef, "ef_search exceeds the stage's max_ef");
    return PA_OK;
}

static int check_mode(pa_stage *st, int mode, int ef, int k) {
    PA_REQUIRE(mode == PA_OUT_HANDOFF || mode == PA_OUT_STAGE2 || mode == PA_OUT_TOPK,
               "mode must be PA_OUT_HANDOFF, PA_OUT_STAGE2 or PA_OUT_TOPK");
    if (mode == PA_OUT_HANDOFF) return PA_OK;
    if (!st->has_refine)
        return fail(PA_ERR_STATE, "the stage has no refinement data (pa_stage_attach_refine)");
    if (mode == PA_OUT_TOPK) {
        if (st->rx.full_nbr == nullptr)
            return fail(PA_ERR_STATE, "top-k output needs the packed full graph");
        PA_REQUIRE(k > 0 && k <= PA_BEAMS * ef, "k must be in (0, 4 * ef_search]");
    }
    return PA_OK;
}

// Row length of a mode's output.
static int64_t out_row(int mode, int ef, int k) {
    return mode == PA_OUT_TOPK ? k : static_cast<int64_t>(PA_BEAMS) * ef;
}

// The refinement of rows [0, n): candidates cand_* [n, 4 * ef] -> out_* (stage-2
// rows or top-k), on `stream`, with the visited slots of stream number `lane`.
static int enqueue_refine(pa_stage *st, const float *rotated, const int64_t *cand_I,
                          const float *cand_D, int64_t *out_I, float *out_D, int64_t n, int ef,
                          int k, int mode, int lane, int32_t *stats, cudaStream_t stream) {
    const pa_stage_index &ix = st->ix;
    return refine_enqueue(out_I, out_D, cand_I, cand_D, rotated, ix.d_model, st->rx.storage_full,
                          ix.packed_nbr, ix.row_of, ix.n_neighbors, st->rx.full_nbr,
                          st->rx.full_degree, n, ix.n_nodes, ix.d_model, ix.d_principle,
                          PA_BEAMS * ef, ef, k, mode == PA_OUT_TOPK ? 3 : 2, st->pool,
                          lane * st->slots_per_stream, st->slots_per_stream, stats, stream);
}

}  // namespace pa

extern "C" int pa_stage_create(pa_stage **out, const pa_stage_index *index, int64_t max_batch,
                               int max_ef, int n_streams) {
    using namespace pa;
    PA_REQUIRE(out != nullptr && index != nullptr, "null pointer");
    *out = nullptr;
    const pa_stage_index &ix = *index;
    PA_REQUIRE(max_batch > 0 && max_batch <= 0x7fffffff, "max_batch out of range");
    PA_REQUIRE(pa_heap_size_for(max_ef) > 0, "max_ef must be in (0, 2048]");
    PA_REQUIRE(n_streams >= 1 && n_streams <= 16, "n_streams must be in [1, 16]");
    PA_REQUIRE(ix.packed_nbr && ix.row_of && ix.storage && ix.entry_nodes && ix.entry_vectors,
               "index pointers missing");
    PA_REQUIRE(ix.d_principle > 0 && ix.d_principle % 4 == 0 && ix.d_model >= ix.d_principle &&
                   ix.d_model % 4 == 0,
               "d_principle / d_model must be multiples of 4 with d_principle <= d_model");
    PA_REQUIRE(ix.n_leaves > 0 && ix.n_leaves % 32 == 0, "n_leaves must be a multiple of 32");
    PA_REQUIRE(ix.route_vectors == nullptr || ix.n_routers > 0, "n_routers must be positive");
    PA_REQUIRE(ix.n_neighbors > 0 && ix.n_neighbors % 32 == 0 && ix.n_neighbors <= 64,
               "n_neighbors must be 32 or 64");
    pa_stage *st = new (std::nothrow) pa_stage();
    if (st == nullptr) return fail(PA_ERR_CUDA, "out of host memory");
    st->ix = ix;
    st->max_batch = max_batch;
    st->max_ef = max_ef;
    cudaError_t e = cudaGetDevice(&st->device);
    auto bail = [&](cudaError_t err, const char *what) {
        pa_stage_destroy(st);
        return cuda_fail(err, what);
    };
    if (e != cudaSuccess) return bail(e, "cudaGetDevice");
    for (int i = 0; i < n_streams; ++i) {
        cudaStream_t s;
        e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
        if (e != cudaSuccess) return bail(e, "cudaStreamCreateWithFlags");
        st->streams.push_back(s);
        cudaEvent_t ev;
        e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e != cudaSuccess) return bail(e, "cudaEventCreateWithFlags");
        st->projected.push_back(ev);
    }
    e = cudaStreamCreateWithFlags(&st->copy_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return bail(e, "cudaStreamCreateWithFlags");
    const size_t B = static_cast<size_t>(max_batch);
    const size_t row = sizeof(float) * ix.d_model;
    const size_t out_elems = B * PA_BEAMS * max_ef;
#define PA_STAGE_ALLOC(ptr, bytes)                                              \
    if ((e = cudaMalloc(reinterpret_cast<void **>(&(ptr)), (bytes))) != cudaSuccess) \
        return bail(e, "cudaMalloc(" #ptr ")")
    PA_STAGE_ALLOC(st->d_raw, B * row);
    if (ix.VT != nullptr) PA_STAGE_ALLOC(st->d_rot, B * row);
    PA_STAGE_ALLOC(st->d_router, B * sizeof(int64_t));
    PA_STAGE_ALLOC(st->d_ep_D, B * ix.n_leaves * sizeof(float));
    PA_STAGE_ALLOC(st->d_ep_I, B * ix.n_leaves * sizeof(int64_t));
    if (ix.route_vectors != nullptr && ix.n_routers > 1) {
        PA_STAGE_ALLOC(st->d_dots, B * ix.n_routers * sizeof(float));
        PA_STAGE_ALLOC(st->d_rnorm, ix.n_routers * sizeof(float));
    }
    PA_STAGE_ALLOC(st->d_out_I, out_elems * sizeof(int64_t));
    PA_STAGE_ALLOC(st->d_out_D, out_elems * sizeof(float));
#undef PA_STAGE_ALLOC
    if (st->d_rnorm != nullptr) {
        int rc = router_norms_launch(st->d_rnorm, ix.route_vectors, ix.n_routers, ix.d_principle,
                                     st->streams[0]);
        if (rc != PA_OK) { pa_stage_destroy(st); return rc; }
        if ((e = cudaStreamSynchronize(st->streams[0])) != cudaSuccess)
            return bail(e, "cudaStreamSynchronize");
    }
    *out = st;
    return PA_OK;
}

extern "C" void pa_stage_destroy(pa_stage *st) {
    if (st == nullptr) return;
    pa::DeviceScope scope;
    scope.enter(st->device);
    for (cudaStream_t s : st->streams) {
        cudaStreamSynchronize(s);
        cudaStreamDestroy(s);
    }
    if (st->copy_stream != nullptr) {
        cudaStreamSynchronize(st->copy_stream);
        cudaStreamDestroy(st->copy_stream);
    }
    for (cudaEvent_t ev : st->projected) cudaEventDestroy(ev);
    cudaFree(st->d_raw);
    cudaFree(st->d_rot);
    cudaFree(st->d_router);
    cudaFree(st->d_ep_D);
    cudaFree(st->d_ep_I);
    cudaFree(st->d_dots);
    cudaFree(st->d_rnorm);
    cudaFree(st->d_out_I);
    cudaFree(st->d_out_D);
    cudaFree(st->d_ref_I);
    cudaFree(st->d_ref_D);
    pa_visited_pool_destroy(st->pool);
    for (cudaEvent_t ev : st->slot_done) cudaEventDestroy(ev);
    cudaFreeHost(st->h_slot_I);
    cudaFreeHost(st->h_slot_D);
    cudaFreeHost(st->h_slot_rot);
    delete st;
}

namespace pa {

// H2D -> project -> route -> traverse [-> refine] -> D2H of rows [lo, lo + m) of a
// host batch, everything on stream number `lane`.  Results go to host_out_* rows
// starting at row `dst_row` (row length: the mode's), the rotated queries (if
// asked for) on the copy stream as soon as they exist.
static int enqueue_host_chunk(pa_stage *st, const float *host_query, float *host_rotated,
                              int64_t *host_out_I, float *host_out_D, int64_t lo, int64_t m,
                              int64_t dst_row, int ef, int k, int mode, int lane) {
    const pa_stage_index &ix = st->ix;
    const int64_t d = ix.d_model;
    const int64_t cand_row = static_cast<int64_t>(PA_BEAMS) * ef;
    const int64_t row = out_row(mode, ef, k);
    cudaStream_t s = st->streams[lane];
    float *raw = st->d_raw + lo * d;
    float *rot = st->d_rot ? st->d_rot + lo * d : nullptr;
    PA_CUDA_TRY(cudaMemcpyAsync(raw, host_query, sizeof(float) * m * d, cudaMemcpyHostToDevice, s));
    int rc = enqueue_chunk(st, raw, rot, st->d_router + lo,
                           st->d_dots ? st->d_dots + lo * ix.n_routers : nullptr,
                           st->d_ep_D + lo * ix.n_leaves, st->d_ep_I + lo * ix.n_leaves,
                           st->d_out_I + lo * cand_row, st->d_out_D + lo * cand_row, m, ef, nullptr,
                           s, st->projected[lane]);
    if (rc != PA_OK) return rc;
    if (host_rotated != nullptr) {
        // the rotated queries travel back on their own stream while the chunk
        // is still routing and traversing
        PA_CUDA_TRY(cudaStreamWaitEvent(st->copy_stream, st->projected[lane], 0));
        PA_CUDA_TRY(cudaMemcpyAsync(host_rotated, rot ? rot : raw, sizeof(float) * m * d,
                                    cudaMemcpyDeviceToHost, st->copy_stream));
    }
    const int64_t *src_I = st->d_out_I + lo * cand_row;
    const float *src_D = st->d_out_D + lo * cand_row;
    if (mode != PA_OUT_HANDOFF) {
        int64_t *ref_I = st->d_ref_I + lo * cand_row;
        float *ref_D = st->d_ref_D + lo * cand_row;
        rc = enqueue_refine(st, rot ? rot : raw, src_I, src_D, ref_I, ref_D, m, ef, k, mode, lane,
                            nullptr, s);
        if (rc != PA_OK) return rc;
        src_I = ref_I;
        src_D = ref_D;
    }
    PA_CUDA_TRY(cudaMemcpyAsync(host_out_I + dst_row * row, src_I, sizeof(int64_t) * m * row,
                                cudaMemcpyDeviceToHost, s));
    PA_CUDA_TRY(cudaMemcpyAsync(host_out_D + dst_row * row, src_D, sizeof(float) * m * row,
                                cudaMemcpyDeviceToHost, s));
    return PA_OK;
}

}  // namespace pa

extern "C" int pa_stage_search_ex(pa_stage *st, const float *host_query, float *host_rotated,
                                  int64_t *host_out_I, float *host_out_D, int64_t batch, int ef,
                                  int k, int mode, int64_t chunk) {
    using namespace pa;
    int rc = check_call(st, batch, ef);
    if (rc != PA_OK) return rc;
    rc = check_mode(st, mode, ef, k);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(host_query && host_out_I && host_out_D, "null host pointer");
    PA_REQUIRE(chunk >= 0, "chunk must not be negative");
    if (chunk == 0 || chunk > batch) chunk = batch;
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    const int64_t d = st->ix.d_model;
    int n = 0;
    for (int64_t lo = 0; lo < batch; lo += chunk, ++n) {
        const int64_t m = (lo + chunk <= batch) ? chunk : batch - lo;
        rc = enqueue_host_chunk(st, host_query + lo * d,
                                host_rotated ? host_rotated + lo * d : nullptr, host_out_I,
                                host_out_D, lo, m, lo, ef, k, mode,
                                n % static_cast<int>(st->streams.size()));
        if (rc != PA_OK) return rc;
    }
    for (cudaStream_t s : st->streams) PA_CUDA_TRY(cudaStreamSynchronize(s));
    PA_CUDA_TRY(cudaStreamSynchronize(st->copy_stream));
    return PA_OK;
}

extern "C" int pa_stage_search(pa_stage *st, const float *host_query, float *host_rotated,
                               int64_t *host_out_I, float *host_out_D, int64_t batch,
                               int ef, int64_t chunk) {
    return pa_stage_search_ex(st, host_query, host_rotated, host_out_I, host_out_D, batch, ef, 0,
                              PA_OUT_HANDOFF, chunk);
}

extern "C" int pa_stage_search_device_ex(pa_stage *st, const float *dev_query, int64_t *dev_out_I,
                                         float *dev_out_D, int64_t batch, int ef, int k, int mode,
                                         int32_t *dev_stats, int32_t *dev_refine_stats) {
    using namespace pa;
    int rc = check_call(st, batch, ef);
    if (rc != PA_OK) return rc;
    rc = check_mode(st, mode, ef, k);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(dev_query && dev_out_I && dev_out_D, "null device pointer");
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    int64_t *cand_I = mode == PA_OUT_HANDOFF ? dev_out_I : st->d_out_I;
    float *cand_D = mode == PA_OUT_HANDOFF ? dev_out_D : st->d_out_D;
    rc = enqueue_chunk(st, dev_query, st->d_rot, st->d_router, st->d_dots, st->d_ep_D, st->d_ep_I,
                       cand_I, cand_D, batch, ef, dev_stats, st->streams[0]);
    if (rc != PA_OK || mode == PA_OUT_HANDOFF) return rc;
    return enqueue_refine(st, st->d_rot ? st->d_rot : dev_query, cand_I, cand_D, dev_out_I,
                          dev_out_D, batch, ef, k, mode, 0, dev_refine_stats, st->streams[0]);
}

extern "C" int pa_stage_search_device(pa_stage *st, const float *dev_query, int64_t *dev_out_I,
                                      float *dev_out_D, int64_t batch, int ef,
                                      int32_t *dev_stats) {
    return pa_stage_search_device_ex(st, dev_query, dev_out_I, dev_out_D, batch, ef, 0,
                                     PA_OUT_HANDOFF, dev_stats, nullptr);
}

// ---- refinement data ---------------------------------------------------------------
extern "C" int pa_stage_attach_refine(pa_stage *st, const pa_refine_index *rx,
                                      int slots_per_stream) {
    using namespace pa;
    if (st == nullptr) return fail(PA_ERR_STATE, "stage is null");
    PA_REQUIRE(rx != nullptr && rx->storage_full != nullptr, "full-dimension vectors missing");
    PA_REQUIRE(rx->full_nbr == nullptr || (rx->full_degree > 0 && rx->full_degree <= 64),
               "full-graph degree must be in (0, 64]");
    PA_REQUIRE(slots_per_stream >= 0, "slots_per_stream must not be negative");
    if (st->has_refine) return fail(PA_ERR_STATE, "refinement data already attached");
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    if (slots_per_stream == 0) {
        // one wave of refinement CTAs: what the device holds at once
        int sms = 0;
        PA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, st->device));
        slots_per_stream = sms * refine_ctas_per_sm(st->ix.d_model);
        if (slots_per_stream > st->max_batch) slots_per_stream = static_cast<int>(st->max_batch);
        // a slot is one byte per node: on a very large index a full wave of slots is not
        // affordable -- keep the pool within a quarter of the free memory (fewer resident
        // queries then, same results)
        size_t free_b = 0, total_b = 0;
        PA_CUDA_TRY(cudaMemGetInfo(&free_b, &total_b));
        const int64_t per_slot = pa_visited_pool_bytes(st->ix.n_nodes, 1) *
                                 static_cast<int64_t>(st->streams.size());
        const int64_t affordable = static_cast<int64_t>(free_b / 4) / (per_slot > 0 ? per_slot : 1);
        if (slots_per_stream > affordable) slots_per_stream = static_cast<int>(affordable < 32 ? 32 : affordable);
    }
    int rc = pa_visited_pool_create(&st->pool, st->ix.n_nodes,
                                    slots_per_stream * static_cast<int>(st->streams.size()));
    if (rc != PA_OK) return rc;
    const size_t elems = static_cast<size_t>(st->max_batch) * PA_BEAMS * st->max_ef;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&st->d_ref_I), elems * sizeof(int64_t));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&st->d_ref_D), elems * sizeof(float));
    if (e != cudaSuccess) {
        pa_visited_pool_destroy(st->pool);
        st->pool = nullptr;
        cudaFree(st->d_ref_I);
        st->d_ref_I = nullptr;
        return cuda_fail(e, "cudaMalloc(refinement output)");
    }
    st->rx = *rx;
    st->slots_per_stream = slots_per_stream;
    st->has_refine = true;
    return PA_OK;
}

// ---- submit / wait: the consumer overlaps the stage --------------------------------
// Upstream's pipeline refines chunk i-2 on the CPU while the GPU traverses chunk
// i-1 (extension/pipeline_cpu.cpp:99-141), with device and pinned buffers it
// allocates in every call (:78-96).  Here a "slot" is one stream of the stage plus
// a share of its device buffers plus pinned host buffers that live as long as the
// stage; submit enqueues a chunk on a slot and returns, wait blocks until that
// chunk's results are in the slot's pinned buffers.
extern "C" int64_t pa_stage_slot_rows(pa_stage *st) {
    return st == nullptr ? 0 : st->max_batch / static_cast<int64_t>(st->streams.size());
}

static int ensure_slots(pa_stage *st) {
    using namespace pa;
    if (st->h_slot_I != nullptr) return PA_OK;
    const int64_t n_slots = static_cast<int64_t>(st->streams.size());
    st->slot_rows = st->max_batch / n_slots;
    PA_REQUIRE(st->slot_rows > 0, "max_batch is smaller than the number of streams");
    const size_t rows = static_cast<size_t>(st->slot_rows * n_slots);
    const size_t out = rows * PA_BEAMS * st->max_ef;
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void **>(&st->h_slot_I), out * sizeof(int64_t),
                                  cudaHostAllocDefault);
    if (e == cudaSuccess)
        e = cudaHostAlloc(reinterpret_cast<void **>(&st->h_slot_D), out * sizeof(float),
                          cudaHostAllocDefault);
    if (e == cudaSuccess)
        e = cudaHostAlloc(reinterpret_cast<void **>(&st->h_slot_rot),
                          rows * st->ix.d_model * sizeof(float), cudaHostAllocDefault);
    for (int64_t i = 0; e == cudaSuccess && i < n_slots; ++i) {
        cudaEvent_t ev;
        e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e == cudaSuccess) st->slot_done.push_back(ev);
    }
    if (e != cudaSuccess) return cuda_fail(e, "pinned slot buffers");
    st->slot_pending.assign(n_slots, -1);
    return PA_OK;
}

extern "C" int pa_stage_submit(pa_stage *st, int slot, const float *host_query, int64_t n, int ef,
                               int k, int mode, int want_rotated) {
    using namespace pa;
    if (st == nullptr) return fail(PA_ERR_STATE, "stage is null");
    PA_REQUIRE(slot >= 0 && slot < static_cast<int>(st->streams.size()), "no such slot");
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    int rc = ensure_slots(st);
    if (rc != PA_OK) return rc;
    PA_REQUIRE(n >= 0 && n <= st->slot_rows, "more queries than a slot holds (pa_stage_slot_rows)");
    PA_REQUIRE(ef > 0 && ef <= st->max_ef, "ef_search exceeds the stage's max_ef");
    rc = check_mode(st, mode, ef, k);
    if (rc != PA_OK) return rc;
    if (st->slot_pending[slot] >= 0)
        return fail(PA_ERR_STATE, "slot %d still holds a chunk: wait for it first", slot);
    PA_REQUIRE(n == 0 || host_query != nullptr, "null host pointer");
    const int64_t cap = st->slot_rows * PA_BEAMS * st->max_ef;
    if (n > 0) {
        rc = enqueue_host_chunk(st, host_query,
                                want_rotated ? st->h_slot_rot + slot * st->slot_rows * st->ix.d_model
                                             : nullptr,
                                st->h_slot_I + slot * cap, st->h_slot_D + slot * cap,
                                slot * st->slot_rows, n, 0, ef, k, mode, slot);
        if (rc != PA_OK) return rc;
        if (want_rotated) {
            // the slot is done when its own stream and the rotated-query copy are
            PA_CUDA_TRY(cudaEventRecord(st->slot_done[slot], st->copy_stream));
            PA_CUDA_TRY(cudaStreamWaitEvent(st->streams[slot], st->slot_done[slot], 0));
        }
    }
    PA_CUDA_TRY(cudaEventRecord(st->slot_done[slot], st->streams[slot]));
    st->slot_pending[slot] = n;
    return PA_OK;
}

extern "C" int pa_stage_wait(pa_stage *st, int slot, int64_t **host_out_I, float **host_out_D,
                             float **host_rotated, int64_t *n_rows) {
    using namespace pa;
    if (st == nullptr) return fail(PA_ERR_STATE, "stage is null");
    PA_REQUIRE(slot >= 0 && slot < static_cast<int>(st->streams.size()), "no such slot");
    if (st->h_slot_I == nullptr || st->slot_pending[slot] < 0)
        return fail(PA_ERR_STATE, "slot %d holds no chunk", slot);
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    PA_CUDA_TRY(cudaEventSynchronize(st->slot_done[slot]));
    const int64_t cap = st->slot_rows * PA_BEAMS * st->max_ef;
    if (host_out_I != nullptr) *host_out_I = st->h_slot_I + slot * cap;
    if (host_out_D != nullptr) *host_out_D = st->h_slot_D + slot * cap;
    if (host_rotated != nullptr) *host_rotated = st->h_slot_rot + slot * st->slot_rows * st->ix.d_model;
    if (n_rows != nullptr) *n_rows = st->slot_pending[slot];
    st->slot_pending[slot] = -1;
    return PA_OK;
}

extern "C" int pa_stage_synchronize(pa_stage *st) {
    if (st == nullptr) return pa::fail(PA_ERR_STATE, "stage is null");
    pa::DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    for (cudaStream_t s : st->streams) PA_CUDA_TRY(cudaStreamSynchronize(s));
    PA_CUDA_TRY(cudaStreamSynchronize(st->copy_stream));
    return PA_OK;
}

extern "C" void *pa_stage_stream(pa_stage *st) {
    return st == nullptr ? nullptr : static_cast<void *>(st->streams[0]);
}

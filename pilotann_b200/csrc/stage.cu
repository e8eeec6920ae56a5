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
    delete st;
}

extern "C" int pa_stage_search(pa_stage *st, const float *host_query, float *host_rotated,
                               int64_t *host_out_I, float *host_out_D, int64_t batch,
                               int ef, int64_t chunk) {
    using namespace pa;
    int rc = check_call(st, batch, ef);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(host_query && host_out_I && host_out_D, "null host pointer");
    PA_REQUIRE(chunk >= 0, "chunk must not be negative");
    if (chunk == 0 || chunk > batch) chunk = batch;
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    const pa_stage_index &ix = st->ix;
    const int64_t d = ix.d_model;
    const int64_t out_row = static_cast<int64_t>(PA_BEAMS) * ef;
    int n = 0;
    for (int64_t lo = 0; lo < batch; lo += chunk, ++n) {
        const int64_t m = (lo + chunk <= batch) ? chunk : batch - lo;
        cudaStream_t s = st->streams[n % st->streams.size()];
        float *raw = st->d_raw + lo * d;
        float *rot = st->d_rot ? st->d_rot + lo * d : nullptr;
        PA_CUDA_TRY(cudaMemcpyAsync(raw, host_query + lo * d, sizeof(float) * m * d,
                                    cudaMemcpyHostToDevice, s));
        rc = enqueue_chunk(st, raw, rot, st->d_router + lo,
                           st->d_dots ? st->d_dots + lo * ix.n_routers : nullptr,
                           st->d_ep_D + lo * ix.n_leaves,
                           st->d_ep_I + lo * ix.n_leaves, st->d_out_I + lo * out_row,
                           st->d_out_D + lo * out_row, m, ef, nullptr, s,
                           st->projected[n % st->streams.size()]);
        if (rc != PA_OK) return rc;
        if (host_rotated != nullptr) {
            // the rotated queries travel back on their own stream while the chunk
            // is still routing and traversing
            PA_CUDA_TRY(cudaStreamWaitEvent(st->copy_stream,
                                            st->projected[n % st->streams.size()], 0));
            PA_CUDA_TRY(cudaMemcpyAsync(host_rotated + lo * d, rot ? rot : raw,
                                        sizeof(float) * m * d, cudaMemcpyDeviceToHost,
                                        st->copy_stream));
        }
        PA_CUDA_TRY(cudaMemcpyAsync(host_out_I + lo * out_row, st->d_out_I + lo * out_row,
                                    sizeof(int64_t) * m * out_row, cudaMemcpyDeviceToHost, s));
        PA_CUDA_TRY(cudaMemcpyAsync(host_out_D + lo * out_row, st->d_out_D + lo * out_row,
                                    sizeof(float) * m * out_row, cudaMemcpyDeviceToHost, s));
    }
    for (cudaStream_t s : st->streams) PA_CUDA_TRY(cudaStreamSynchronize(s));
    PA_CUDA_TRY(cudaStreamSynchronize(st->copy_stream));
    return PA_OK;
}

extern "C" int pa_stage_search_device(pa_stage *st, const float *dev_query, int64_t *dev_out_I,
                                      float *dev_out_D, int64_t batch, int ef,
                                      int32_t *dev_stats) {
    using namespace pa;
    int rc = check_call(st, batch, ef);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(dev_query && dev_out_I && dev_out_D, "null device pointer");
    DeviceScope scope;
    PA_CUDA_TRY(scope.enter(st->device));
    return enqueue_chunk(st, dev_query, st->d_rot, st->d_router, st->d_dots, st->d_ep_D,
                         st->d_ep_I,
                         dev_out_I, dev_out_D, batch, ef, dev_stats, st->streams[0]);
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

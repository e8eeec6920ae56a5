/*
 * pilotann_b200.h -- C ABI of the B200 (sm_100a) GPU search stage.
 *
 * Plain pointers and sizes only; no torch / C++ types.  Every pointer is a
 * DEVICE pointer on the current CUDA device unless its name starts with
 * "host_".  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * All calls are asynchronous on `stream` unless stated otherwise and return 0
 * (PA_OK) or a negative error code; pa_last_error() gives the message of the
 * last failure on the calling thread.  The library never falls back to the
 * CPU: without a usable CUDA device every compute call fails with
 * PA_ERR_CUDA.
 *
 * "Upstream" below = the PilotANN reference repository; paths are relative to
 * its root.  The Python binding that mirrors the upstream pybind11 module over
 * this ABI is pilotann_b200/extension.py.
 */
#ifndef PILOTANN_B200_H
#define PILOTANN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_OK 0
#define PA_ERR_ARG (-1)        /* a shape / size / alignment the call rejects */
#define PA_ERR_CUDA (-2)       /* a CUDA runtime call or a launch failed */
#define PA_ERR_UNPACKABLE (-3) /* pa_pack_graph: input cannot be represented */
#define PA_ERR_STATE (-4)      /* stage object used out of order */

#define PA_BEAMS 4             /* beams per query, traverse_cuda.cu:13 */

int pa_version(void);
const char *pa_last_error(void);

/* Heap capacity the traversal uses for a given ef_search (32/64/128/256), or
 * -1 if ef_search is outside (0, 2048].  Upstream: traverse_cuda.cu:302-315. */
int pa_heap_size_for(int ef_search);

/* ---- traversal, upstream tensor layout --------------------------------
 * Replaces `traverse_cuda` (extension/traverse_cuda.cu:249-315, declared in
 * extension/entry.cpp:32-38): multi-beam search of a batch of queries over the
 * sampled sub-graph in the reduced space.
 *   output_I [batch,4,ef] int64, output_D [batch,4,ef] f32: per beam, worst ->
 *     best; (-1,+inf) pads first when a beam holds fewer than ef results,
 *     (-1,-inf) tail when ef > 256.
 *   indptr [n_nodes+1], indices [*], mapping [n_nodes] int64 (CSR over global
 *     ids, -1 padded rows; mapping = row of `storage` or -1)
 *   storage [n_storage,d_model] f32, query [batch,d_model] f32
 *   initial_I / initial_D [batch,n_initials]: entry ids and their reduced
 *     squared distances.
 *   stats: NULL, or int32 [batch,4] = rounds, expanded nodes, distance
 *     evaluations, bloom bits set.
 * Rejects (PA_ERR_ARG) what upstream rejects: n_neighbors % 32 != 0,
 * 4*n_neighbors > 256, ef_search > 2048; and d_model % 4 != 0 or pointers not
 * 16-byte aligned (upstream would fault on those). */
int pa_traverse_csr(int64_t *output_I, float *output_D, const int64_t *indptr,
                    const int64_t *indices, const int64_t *mapping,
                    const float *storage, const float *query,
                    const int64_t *initial_I, const float *initial_D,
                    int64_t batch, int64_t n_nodes, int64_t n_storage,
                    int d_model, int n_neighbors, int n_initials, int ef_search,
                    int32_t *stats, void *stream);

/* ---- packed device-resident index --------------------------------------
 * Counterpart of the device copies `IndexStaged.to` prepares
 * (pilot_ann/layers/staged.py:124-139), laid out for one dependent load per
 * hop: packed_nbr [n_storage, n_neighbors][4] int32, indexed by storage row --
 * per neighbour slot {global id, storage row, two words of bloom probes: the
 * four 15-bit hash positions of the id (upstream bloom.cuh:9-16 chained as in
 * traverse_cuda.cu:60-74) and, per hash step, whether the slot is the first of
 * its 32-slot chunk to touch that bit} -- and row_of [n_nodes] int32
 * (= mapping).  packed_nbr takes 16 * n_storage * n_neighbors bytes and must be
 * 16-byte aligned.
 * Fails with PA_ERR_UNPACKABLE (after a stream synchronise) if a node with a
 * non-empty adjacency row has no storage row, or an id does not fit int32.
 * Synchronous. */
int pa_pack_graph(int32_t *packed_nbr, int32_t *row_of, const int64_t *indptr,
                  const int64_t *indices, const int64_t *mapping, int64_t n_nodes,
                  int64_t n_storage, int n_neighbors, void *stream);

/* Same search as pa_traverse_csr, same outputs bit for bit, over the packed
 * index (the fast path used by the stage object and the Python layers). */
int pa_traverse_packed(int64_t *output_I, float *output_D,
                       const int32_t *packed_nbr, const int32_t *row_of,
                       const float *storage, const float *query,
                       const int64_t *initial_I, const float *initial_D,
                       int64_t batch, int64_t n_nodes, int64_t n_storage,
                       int d_model, int n_neighbors, int n_initials,
                       int ef_search, int32_t *stats, void *stream);

/* ---- entry routing (FES) -----------------------------------------------
 * Replaces `routing_cuda` (extension/routing_cuda.cu:70-113, entry.cpp:59-62)
 * and the id gather that follows it in IndexEntry.search
 * (pilot_ann/layers/entry.py:81-88).
 *   router [batch] int64: nearest router of each query (exact order; ties ->
 *     lowest index)
 *   leaf_D [batch,n_leaves] f32: squared distances to that router's leaves
 *   leaf_I: NULL, or [batch,n_leaves] int64 = entry_nodes[router[b], :]
 *   route_vectors [n_routers,d], entry_nodes [n_routers,n_leaves] int64,
 *   entry_vectors [n_routers,n_leaves,d] f32.
 * n_leaves % 32 == 0 as upstream (routing_cuda.cu:90); d % 4 == 0. */
int pa_route(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
             const float *route_vectors, const int64_t *entry_nodes,
             const float *entry_vectors, int64_t batch, int d_model,
             int n_routers, int n_leaves, void *stream);

/* Same result as pa_route, bit for bit, with the dense query x router part on the
 * tensor cores (tcgen05, fp32-grade three-product TF32): the tensor-core scores
 * shortlist the routers, the shortlisted ones are re-measured exactly.
 * workspace: device memory of pa_route_workspace_floats(batch, n_routers) floats,
 * 16-byte aligned; NULL falls back to pa_route. */
int64_t pa_route_workspace_floats(int64_t batch, int n_routers);
int pa_route_ws(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
                const float *route_vectors, const int64_t *entry_nodes,
                const float *entry_vectors, int64_t batch, int d_model, int n_routers,
                int n_leaves, float *workspace, void *stream);

/* ---- query projection ---------------------------------------------------
 * Replaces the CPU `query @ VT.T` of IndexStaged.search
 * (pilot_ann/layers/staged.py:198): out[b, j] = sum_k query[b,k] * VT[j,k] for
 * j < d_out.  query [batch,d_model], VT [>= d_out, d_model] row-major, out
 * [batch, ld_out] with ld_out >= d_out. */
int pa_project(float *out, const float *query, const float *VT, int64_t batch,
               int d_model, int d_out, int64_t ld_out, void *stream);

/* Synchronises the current device and returns 0, or 1 if a tensor-core kernel of
 * this library gave up on a bounded wait since the last reset (its output is
 * then undefined), or PA_ERR_CUDA.  No upstream counterpart. */
int pa_device_status(int reset);

/* Diagnostic for the bounded waits: launches one thread that polls 16 times on an
 * mbarrier phase nothing completes, gives up, and sets the status word the way a
 * tensor-core kernel of this library does when a copy never lands.  Afterwards
 * pa_device_status(1) returns 1 and the device is as usable as before.  While the
 * word is set, entry routing ignores tensor-core router scores and measures every
 * router exactly.  No upstream counterpart. */
int pa_selftest_bounded_wait(void *stream);

/* ---- visited-set pool -------------------------------------------------------
 * Device counterpart of upstream's `Bitmask` / `BitmaskPool`
 * (extension/inc/bitmask.hpp:12-45, 51-76; used at traverse_cpu.cpp:196-200 and
 * 297-312): per worker an array of epoch markers over all nodes, so that the
 * visited state of a query never needs clearing.  A worker here is a resident
 * CTA of the refinement kernel; slot i belongs to CTA i of a launch, one byte per
 * node, markers 1..254, wiped on wrap-around.  Allocates
 * pa_visited_pool_bytes(n_nodes, n_slots) bytes of device memory once.  Launches
 * that may overlap on the GPU must not share a pool (the stage object gives each
 * of its streams its own slots). */
typedef struct pa_visited_pool pa_visited_pool;
int64_t pa_visited_pool_bytes(int64_t n_nodes, int n_slots);
int pa_visited_pool_create(pa_visited_pool **out, int64_t n_nodes, int n_slots);
void pa_visited_pool_destroy(pa_visited_pool *pool);
int pa_visited_pool_slots(const pa_visited_pool *pool);

/* ---- refinement on the GPU ---------------------------------------------------
 * Replaces the CPU consumer of the handoff, `traverse_refine`
 * (extension/traverse_cpu.cpp:261-369, declared in extension/entry.cpp:39-46),
 * i.e. two calls of `traverse_cpu_kernel` (traverse_cpu.cpp:12-163) per query:
 * stage 2 on the sampled sub-graph (distances completed over dims d_principle ..
 * d_model, REFINE_STEP = 2 expansions, result written back over the handoff row)
 * and stage 3 on the full graph (top-k).  Heap capacity H follows upstream's CPU
 * dispatch (traverse_cpu.cpp:228-254): pa_cpu_heap_size_for(ef_search).
 *   cand_I / cand_D [batch, n_cand]: the handoff as pa_traverse_* wrote it
 *     (n_cand = 4 * ef_search), read only
 *   query [batch, d_model]: the full rotated queries
 *   storage_full [n_nodes, d_model] f32
 *   packed_nbr / row_of / n_neighbors: the packed sub-graph (pa_pack_graph)
 *   full_nbr [n_nodes, full_degree] int32: pa_pack_fullgraph (stages == 3 only)
 *   stages 2: out_I / out_D [batch, n_cand] <- the stage-2 row (what upstream leaves
 *     in the handoff buffer: H best ascending behind (-1, -inf) pads);
 *   stages 3: out_I [batch, k] int64, out_D [batch, k] f32 <- top-k ascending.
 *   stats: NULL or int32 [batch, 4] = stage-2 expansions, stage-2 distance
 *     evaluations, stage-3 expansions, stage-3 evaluations.
 * Distances are summed in this kernel's own order (see csrc/refine.cu); against
 * upstream's AVX2 build they agree within 1e-5 relative. */
int pa_cpu_heap_size_for(int ef_search);
/* Refinement CTAs (one query each) an SM holds at once for vectors of d_model floats:
 * the visited slots worth having per SM.  The counterpart upstream is the size of its
 * BitmaskPool, one bitmask per OpenMP thread (traverse_cpu.cpp:208-226). */
int pa_refine_ctas_per_sm(int d_model);
int pa_pack_fullgraph(int32_t *full_nbr, const int64_t *indptr, const int64_t *indices,
                      int64_t n_nodes, int degree, void *stream);
int pa_refine(int64_t *out_I, float *out_D, const int64_t *cand_I, const float *cand_D,
              const float *query, const float *storage_full, const int32_t *packed_nbr,
              const int32_t *row_of, int n_neighbors, const int32_t *full_nbr,
              int full_degree, int64_t batch, int64_t n_nodes, int d_model,
              int d_principle, int n_cand, int ef_search, int k, int stages,
              pa_visited_pool *pool, int32_t *stats, void *stream);

/* ---- search stage object -------------------------------------------------
 * Replaces the GPU half of `pipeline` (extension/pipeline_cpu.cpp:32-145): its
 * static stream pool (:67-75), the per-call device and pinned handoff buffers
 * (:78-96) and the chunked launch + asynchronous copy-back loop (:120-140).
 * One object per device, created once, reused for every batch. */
typedef struct pa_stage pa_stage;

typedef struct pa_stage_index {
    const int32_t *packed_nbr;   /* pa_pack_graph output */
    const int32_t *row_of;
    const float *storage;        /* [n_storage, d_principle] */
    const float *VT;             /* [d_model, d_model] or NULL (no projection) */
    const float *route_vectors;  /* NULL for the 'random' entry method */
    const int64_t *entry_nodes;  /* [n_routers, n_leaves] or [n_leaves] */
    const float *entry_vectors;  /* [n_routers, n_leaves, d_p] or [n_leaves, d_p] */
    int64_t n_nodes, n_storage;
    int d_model, d_principle, n_neighbors, n_routers, n_leaves;
} pa_stage_index;

/* max_batch = largest batch a call will pass, max_ef = largest ef_search. */
int pa_stage_create(pa_stage **out, const pa_stage_index *index, int64_t max_batch,
                    int max_ef, int n_streams);
void pa_stage_destroy(pa_stage *stage);

/* One pass of the stage over a batch held in HOST memory:
 *   host_query [batch, d_model] f32 (raw, unrotated when index.VT != NULL)
 *   host_rotated: NULL, or [batch, d_model] f32 <- full rotated queries (what
 *     the CPU refinement needs)
 *   host_out_I [batch, 4*ef] int64, host_out_D [batch, 4*ef] f32 <- the
 *     candidate handoff, rows in the layout `traverse_refine` consumes
 *     (pipeline_cpu.cpp:90-95).
 * The batch is cut into `chunk` queries (0 = one chunk); chunks alternate
 * between the stage's streams so that copy-in, kernels and copy-back overlap.
 * Blocks until the handoff is complete.  Host buffers should be pinned. */
int pa_stage_search(pa_stage *stage, const float *host_query, float *host_rotated,
                    int64_t *host_out_I, float *host_out_D, int64_t batch,
                    int ef_search, int64_t chunk);

/* Device-resident variant (inputs already in HBM, outputs stay there);
 * asynchronous on the stage's first stream; dev_query is the raw query.
 * dev_stats may be NULL. Returns after enqueueing. */
int pa_stage_search_device(pa_stage *stage, const float *dev_query,
                           int64_t *dev_out_I, float *dev_out_D, int64_t batch,
                           int ef_search, int32_t *dev_stats);
/* ---- refinement inside the stage ---------------------------------------------
 * With refinement data attached the stage can go on where the handoff used to
 * leave the GPU: the candidates stay in HBM and pa_refine's kernel consumes them
 * on the same stream.  What a call returns is chosen by `mode`:
 *   PA_OUT_HANDOFF  [batch, 4*ef]  the traversal's candidates (pa_stage_search)
 *   PA_OUT_STAGE2   [batch, 4*ef]  the rows after the sub-graph stage of
 *                                  `traverse_refine` (traverse_cpu.cpp:317-326):
 *                                  feed them to upstream `traverse_cpu` for stage 3
 *   PA_OUT_TOPK     [batch, k]     both stages: the final top-k, ascending
 * pa_stage_attach_refine allocates, once: the stage's visited pool
 * (slots_per_stream slots for each stream; 0 = one wave of CTAs) and the device
 * buffers of the refined rows.  storage_full / full_nbr are borrowed.  full_nbr
 * may be NULL when only PA_OUT_STAGE2 is wanted. */
#define PA_OUT_HANDOFF 0
#define PA_OUT_STAGE2 1
#define PA_OUT_TOPK 2
typedef struct pa_refine_index {
    const float *storage_full;   /* [n_nodes, d_model] rotated full vectors */
    const int32_t *full_nbr;     /* [n_nodes, full_degree] pa_pack_fullgraph, or NULL */
    int full_degree;
} pa_refine_index;
int pa_stage_attach_refine(pa_stage *stage, const pa_refine_index *refine,
                           int slots_per_stream);
/* pa_stage_search / pa_stage_search_device with a choice of output; k is used by
 * PA_OUT_TOPK only.  dev_refine_stats: NULL or int32 [batch, 4] as pa_refine. */
int pa_stage_search_ex(pa_stage *stage, const float *host_query, float *host_rotated,
                       int64_t *host_out_I, float *host_out_D, int64_t batch,
                       int ef_search, int k, int mode, int64_t chunk);
int pa_stage_search_device_ex(pa_stage *stage, const float *dev_query,
                              int64_t *dev_out_I, float *dev_out_D, int64_t batch,
                              int ef_search, int k, int mode, int32_t *dev_stats,
                              int32_t *dev_refine_stats);

/* ---- submit / wait ---------------------------------------------------------------
 * Replaces the software pipeline of upstream `pipeline`
 * (extension/pipeline_cpu.cpp:99-141: the CPU refines chunk i-2 while the GPU
 * traverses chunk i-1) without its per-call buffers (:78-96).  The stage has one
 * slot per stream; a slot takes up to pa_stage_slot_rows() queries.
 * pa_stage_submit copies the chunk in, enqueues the kernels of `mode` and the
 * copy back into the slot's own pinned host buffers, and returns; pa_stage_wait
 * blocks until that chunk is complete and hands out the slot's buffers
 * (host_out_* rows of the mode's length, host_rotated [n, d_model] when the
 * submit asked for the rotated queries), valid until the slot's next submit.
 * The pinned buffers are allocated by the first submit and live as long as the
 * stage.  One thread drives a stage. */
int64_t pa_stage_slot_rows(pa_stage *stage);
int pa_stage_submit(pa_stage *stage, int slot, const float *host_query, int64_t n,
                    int ef_search, int k, int mode, int want_rotated);
int pa_stage_wait(pa_stage *stage, int slot, int64_t **host_out_I, float **host_out_D,
                  float **host_rotated, int64_t *n_rows);

int pa_stage_synchronize(pa_stage *stage);
/* cudaStream_t of the stage's first stream (for event timing by the caller). */
void *pa_stage_stream(pa_stage *stage);
/* ---- search without any allocation -----------------------------------------
 * No counterpart upstream (upstream allocates in every call: torch::zeros /
 * torch::empty in routing_cuda.cu:96-98 and pipeline_cpu.cpp:78-96).  For callers
 * that cannot allocate device memory at all: processes that gave the whole GPU to
 * their own memory pool at start-up, and latency-critical threads that must not
 * trigger the device-wide synchronisation cudaMalloc / cudaFree imply.
 *
 * Entry routing followed by traversal over the packed index, i.e. pa_route then
 * pa_traverse_packed, with the intermediate entry tables kept in a static device
 * array of PA_NOALLOC_SCRATCH_BYTES that every GPU loading the library holds
 * until exit.  The caller passes inputs and outputs only: query [batch,
 * d_principle] (already projected / reduced), outputs as pa_traverse_packed.
 * route_vectors may be NULL (shared entry list, n_routers ignored).
 *
 * Limits: batch <= PA_NOALLOC_MAX_BATCH and n_leaves <= PA_NOALLOC_MAX_LEAVES,
 * otherwise PA_ERR_ARG with a message naming the limit.  The call performs no
 * cudaMalloc / cudaFree and calls no allocating library routine.  The first call
 * on each device looks the array's address up (cudaGetSymbolAddress); make that
 * first call before any stream capture.  All calls on a device share the one
 * array, which keeps the previous call's contents (nothing in it needs to start
 * at zero: the routing step overwrites every element the traversal reads);
 * calls that overlap on the GPU -- different streams, or different host threads
 * -- race on it, so serialise them. */
#define PA_NOALLOC_MAX_BATCH 1024
#define PA_NOALLOC_MAX_LEAVES 64
#define PA_NOALLOC_SCRATCH_BYTES (PA_NOALLOC_MAX_BATCH * PA_NOALLOC_MAX_LEAVES * 12)
int pa_search_reduced_noalloc(int64_t *output_I, float *output_D,
                              const int32_t *packed_nbr, const int32_t *row_of,
                              const float *storage, const float *query,
                              const float *route_vectors, const int64_t *entry_nodes,
                              const float *entry_vectors, int64_t batch,
                              int64_t n_nodes, int64_t n_storage, int d_principle,
                              int n_neighbors, int n_routers, int n_leaves,
                              int ef_search, void *stream);

/* Kernels launched by this library on behalf of the calling process. */
int64_t pa_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PILOTANN_B200_H */

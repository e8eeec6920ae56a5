// Shared declarations of the sm_100a search-stage library: error plumbing,
// launchers shared between translation units, the constants with search
// semantics and the bloom hash.
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "pilotann_b200.h"

namespace pa {

// ---- host-side error plumbing (api.cu) -----------------------------------
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t err, const char *what);
void count_launch(int n = 1);

#define PA_CUDA_TRY(expr)                                         \
    do {                                                          \
        cudaError_t err__ = (expr);                               \
        if (err__ != cudaSuccess) return pa::cuda_fail(err__, #expr); \
    } while (0)

#define PA_REQUIRE(cond, ...)                                     \
    do {                                                          \
        if (!(cond)) return pa::fail(PA_ERR_ARG, __VA_ARGS__);    \
    } while (0)

// ---- launchers shared between translation units (used by stage.cu) -------
int traverse_packed_launch(int64_t *output_I, float *output_D, const int32_t *packed_nbr,
                           const int32_t *row_of, const float *storage, const float *query,
                           int64_t ldq, const int64_t *initial_I, const float *initial_D,
                           int64_t batch, int64_t n_nodes, int64_t n_storage, int d_model,
                           int n_neighbors, int n_initials, int ef_search, int32_t *stats,
                           cudaStream_t stream);
int traverse_packed_check(const int64_t *output_I, const float *output_D,
                          const int32_t *packed_nbr, const int32_t *row_of, const float *storage,
                          const float *query, int64_t ldq, const int64_t *initial_I,
                          const float *initial_D, int64_t batch, int64_t n_nodes, int d_model,
                          int n_neighbors, int n_initials, int ef_search);
int route_launch(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
                 int64_t ldq, const float *route_vectors, const int64_t *entry_nodes,
                 const float *entry_vectors, int64_t batch, int d, int n_routers, int n_leaves,
                 float *dots_ws, const float *rnorm2, cudaStream_t stream);
int router_norms_launch(float *rnorm2, const float *route_vectors, int n_routers, int d,
                        cudaStream_t stream);
int gemm_tf32x3_launch(float *out, const float *A, const float *B, int M, int N, int K,
                       int64_t lda, int64_t ldb, int64_t ldo, cudaStream_t stream);
const int *gemm_status_address();
int project_launch(float *out, const float *query, const float *VT, int64_t batch, int d,
                   int d_out, int64_t ld_out, cudaStream_t stream);

void pool_view(const pa_visited_pool *pool, uint8_t **marks, int32_t **epoch, int64_t *slot_stride,
               int *n_slots, int64_t *n_nodes);

int refine_ctas_per_sm(int d_model);
int refine_enqueue(int64_t *out_I, float *out_D, const int64_t *cand_I, const float *cand_D,
                   const float *query, int64_t ldq, const float *storage_full,
                   const int32_t *packed_nbr, const int32_t *row_of, int n_neighbors,
                   const int32_t *full_nbr, int full_degree, int64_t batch, int64_t n_nodes,
                   int d_model, int d_principle, int n_cand, int ef_search, int k, int stages,
                   const pa_visited_pool *pool, int slot_begin, int slot_count, int32_t *stats,
                   cudaStream_t stream);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- constants with search semantics (upstream traverse_cuda.cu:7-15) ----
constexpr int kBeams = PA_BEAMS;        // BEAM_WIDTH
constexpr int kTeam = 8;                // TEAM_SIZE: lanes per distance
constexpr int kTeamsPerWarp = 4;        // N_WORKERS
constexpr int kMaxSlots = 256;          // BUFFER_SIZE
constexpr uint32_t kBloomBits = 32768;  // BITMASK_SIZE
constexpr int kBloomWords = kBloomBits / 32;
constexpr int kFnvSteps = 4;            // FNV_STEP
constexpr uint32_t kFnvPrime = 0x01000193u;
constexpr uint32_t kFnvOffset = 0x811c9dc5u;
constexpr int kEmptyRowTag = -2;       // first pair of a packed row without adjacency
constexpr int kDupTag = -3;            // a slot whose id repeats an earlier slot of its row

// upstream bloom.cuh:9-16: the whole shifted word is xor-ed in at every step
__host__ __device__ __forceinline__ uint32_t fnv1a_32(uint32_t x, uint32_t h) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h ^= x >> (8 * i);
        h *= kFnvPrime;
    }
    return h;
}

// ---- bloom probes of a chunk of 32 neighbour slots -----------------------------
// The filter is tested-and-set 32 slots at a time, the four hash steps in lock
// step, and within a step lanes hitting the same bit are served in ascending
// lane order: only the first ("elected") lane performs the atomic, the others
// have a lower lane setting the very same bit in the same step and see it as
// set.  Positions and elections depend on the 32 ids alone, so the packed index
// stores them next to the ids; for upstream's CSR tensors they are computed on
// the fly.
struct BloomProbe {
    uint32_t pos[kFnvSteps];
    uint32_t elected;  // bit s: this lane performs the atomic of step s
};

#ifdef __CUDACC__
// All 32 lanes of the warp call this together; v < 0 marks a slot without a node.
__device__ __forceinline__ BloomProbe bloom_prepare(int32_t v, int lane) {
    BloomProbe p;
    const bool valid = v >= 0;
    uint32_t h = kFnvOffset;
    p.elected = 0;
#pragma unroll
    for (int s = 0; s < kFnvSteps; ++s) {
        h = fnv1a_32(static_cast<uint32_t>(v), h);
        p.pos[s] = h & (kBloomBits - 1);
        // lanes without a node get a key no node can have
        const uint32_t key = valid ? p.pos[s] : (0x80000000u | lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid && (peers & ((1u << lane) - 1u)) == 0) p.elected |= 1u << s;
    }
    return p;
}
#endif

// Two words per probe: positions are 15 bits each, the election bits ride on top.
__host__ __device__ __forceinline__ uint2 probe_pack(const BloomProbe &p) {
    return make_uint2(p.pos[0] | (p.pos[1] << 15) | ((p.elected & 3u) << 30),
                      p.pos[2] | (p.pos[3] << 15) | ((p.elected >> 2) << 30));
}
__host__ __device__ __forceinline__ BloomProbe probe_unpack(uint2 w) {
    BloomProbe p;
    p.pos[0] = w.x & 0x7fffu; p.pos[1] = (w.x >> 15) & 0x7fffu;
    p.pos[2] = w.y & 0x7fffu; p.pos[3] = (w.y >> 15) & 0x7fffu;
    p.elected = (w.x >> 30) | ((w.y >> 30) << 2);
    return p;
}
static_assert(kBloomBits == (1u << 15), "probe_pack stores 15-bit positions");

}  // namespace pa

// Multi-beam graph traversal in the reduced space -- the HBM-gather-bound hot
// loop of the search stage.  One CTA of four warps per query, one warp per
// beam, as in upstream extension/traverse_cuda.cu:45-246; the search semantics
// (heap layouts, bloom hashing, dealing of candidates to beams, stop rules,
// output order) are upstream's, executed in ONE fixed interleaving so that the
// result is a deterministic function of the inputs:
//   * the bloom filter is cleared, then seeded with the entries, then used;
//   * in a round, beams test-and-set their neighbours in the order beam 0..3
//     (a token passed over named barriers); a beam handles 32 neighbours at a
//     time, running the four hash steps in lock step, and within a step lanes
//     hitting the same bit are served in ascending lane order
//     (__match_any_sync picks the first lane, the others see the bit as set);
//   * each beam's heaps are touched by one lane only.
//
// Two index layouts are served by the same kernel body:
//   CsrLayout    -- upstream's tensors as they are (int64 indptr / indices /
//                   mapping): four dependent loads per hop, kept for drop-in use;
//   PackedLayout -- int32 {global id, storage row} neighbour pairs indexed by
//                   storage row, the row carried through the open heap: two
//                   dependent loads per hop (neighbour row, vector rows).
#include "pa_common.cuh"

namespace pa {

struct OpenVal {
    int32_t node;  // global id, -1 = empty
    int32_t row;   // storage row of `node` (packed layout), -1 = none
};

struct CsrLayout {
    static constexpr bool kPacked = false;
    const int64_t *indptr;
    const int64_t *indices;
    const int64_t *mapping;
    const float *storage;
    int64_t n_nodes;
};

struct PackedLayout {
    static constexpr bool kPacked = true;
    const int2 *nbr;        // [n_storage, n_nb] {global id, storage row}
    const int32_t *row_of;  // [n_nodes]
    const float *storage;
    int64_t n_nodes;
};

constexpr int kThreads = kBeams * 32;

__device__ __forceinline__ void named_sync(int id, int n) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int n) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory");
}

// upstream traverse_cuda.cu:18-43: eight lanes, lane t owns floats
// [32m + 4t, 32m + 4t + 4); acc += fma(dx,dx,dy*dy); acc += fma(dz,dz,dw*dw);
// then the width-8 shuffle tree 4, 2, 1.  Result valid in the team's lane 0.
__device__ __forceinline__ float team_distance(const float *__restrict__ row,
                                               const float *__restrict__ q, int d, int t8,
                                               bool pred) {
    float acc = 0.0f;
    if (pred) {
        for (int off = 4 * t8; off < d; off += 32) {
            float4 p = __ldg(reinterpret_cast<const float4 *>(row + off));
            float4 c = *reinterpret_cast<const float4 *>(q + off);
            float dx = __fsub_rn(c.x, p.x), dy = __fsub_rn(c.y, p.y);
            float dz = __fsub_rn(c.z, p.z), dw = __fsub_rn(c.w, p.w);
            acc = __fadd_rn(acc, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
            acc = __fadd_rn(acc, __fmaf_rn(dz, dz, __fmul_rn(dw, dw)));
        }
    }
#pragma unroll
    for (int off = kTeam / 2; off > 0; off >>= 1)
        acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, off, kTeam));
    return acc;
}

// One chunk of 32 neighbours of one beam: test-and-set in the fixed order.
// Returns true for lanes whose node was already present (or is invalid).
__device__ __forceinline__ bool bloom_visit(uint32_t *bloom, int32_t v, int lane) {
    const bool valid = v >= 0;
    uint32_t pos[kFnvSteps];
    uint32_t h = kFnvOffset;
#pragma unroll
    for (int s = 0; s < kFnvSteps; ++s) {
        h = fnv1a_32(static_cast<uint32_t>(v), h);
        pos[s] = h & (kBloomBits - 1);
    }
    bool found = true;
#pragma unroll
    for (int s = 0; s < kFnvSteps; ++s) {
        // invalid lanes get a key no valid lane can have
        uint32_t key = valid ? pos[s] : (0x80000000u | lane);
        uint32_t peers = __match_any_sync(0xffffffffu, key);
        bool leader = (__ffs(peers) - 1) == lane;
        if (valid && leader) {
            uint32_t bit = 1u << (pos[s] & 31);
            uint32_t old = atomicOr(&bloom[pos[s] >> 5], bit);
            found = found && (old & bit);
        }
        // non-leaders: a lower lane sets this very bit in this step -> seen as set
        __syncwarp();
    }
    return found || !valid;
}

template <int H, class Layout>
__global__ void __launch_bounds__(kThreads)
traverse_kernel(Layout L, int64_t *__restrict__ out_I, float *__restrict__ out_D,
                const float *__restrict__ query, const int64_t *__restrict__ init_I,
                const float *__restrict__ init_D, int d, int64_t ldq, int n_nb, int n_init,
                int ef, int32_t *__restrict__ stats) {
    __shared__ uint32_t bloom[kBloomWords];
    __shared__ float open_key[kBeams][H];
    __shared__ OpenVal open_val[kBeams][H];
    __shared__ float res_key[kBeams][H];
    __shared__ int32_t res_id[kBeams][H];
    __shared__ int2 slots[kMaxSlots];
    __shared__ int counts[kBeams];
    __shared__ int stat_s[4];
    extern __shared__ __align__(16) float q_s[];

    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t b = blockIdx.x;
    const int chunks = n_nb >> 5;  // 1 or 2

    for (int i = threadIdx.x; i < kBloomWords; i += kThreads) bloom[i] = 0;
    for (int i = threadIdx.x; i < d; i += kThreads) q_s[i] = query[b * ldq + i];
    for (int i = lane; i < H; i += 32) {
        open_key[w][i] = CUDART_INF_F;
        open_val[w][i] = OpenVal{-1, -1};
        res_key[w][i] = -CUDART_INF_F;
        res_id[w][i] = -1;
    }
    if (threadIdx.x < 4) stat_s[threadIdx.x] = 0;
    __syncthreads();

    float *okey = open_key[w];
    OpenVal *oval = open_val[w];
    float *rkey = res_key[w];
    int32_t *rid = res_id[w];
    int n_expand = 0, n_eval = 0, n_rounds = 0;

    // ---- entries: entry i belongs to beam i mod 4 (traverse_cuda.cu:96-111).
    // Loads are lane-parallel, the heap inserts run on lane 0 in entry order.
    for (int base = 0; base * kBeams + w < n_init; base += 32) {
        int i = (base + lane) * kBeams + w;
        int64_t node = -1;
        float dist = 0.0f;
        int32_t row = -1;
        if (i < n_init) {
            node = init_I[b * n_init + i];
            dist = init_D[b * n_init + i];
            if constexpr (Layout::kPacked) {
                if (node >= 0 && node < L.n_nodes) row = __ldg(L.row_of + node);
            }
        }
        int todo = min(32, (n_init - w - base * kBeams + kBeams - 1) / kBeams);
        for (int j = 0; j < todo; ++j) {
            int64_t nj = __shfl_sync(0xffffffffu, node, j);
            float dj = __shfl_sync(0xffffffffu, dist, j);
            int32_t rj = __shfl_sync(0xffffffffu, row, j);
            if (lane == 0 && nj >= 0 && !(dj >= -rkey[0])) {
                heap_replace(okey, oval, H, dj, OpenVal{static_cast<int32_t>(nj), rj});
                heap_pushpop(rkey, rid, H, -dj, static_cast<int32_t>(nj));
                uint32_t h = kFnvOffset;
#pragma unroll
                for (int s = 0; s < kFnvSteps; ++s) {
                    h = fnv1a_32(static_cast<uint32_t>(nj), h);
                    uint32_t p = h & (kBloomBits - 1);
                    atomicOr(&bloom[p >> 5], 1u << (p & 31));
                }
            }
        }
    }
    __syncthreads();

    // ---- rounds (traverse_cuda.cu:179-226) ----------------------------------
    for (int step = 0; step < ef; ++step) {
        ++n_rounds;
        // pop until a node with an adjacency row turns up (:118-134)
        int32_t v0 = -1, v1 = -1, r0 = -1, r1 = -1;  // this lane's neighbours
        bool expanding = false;
        for (;;) {
            float key = 0.0f;
            OpenVal val{-1, -1};
            if (lane == 0) {
                heap_pop(okey, oval, H, OpenVal{-1, -1}, key, val);
                if (val.node >= 0 && key >= -rkey[0]) val.node = -1;
            }
            int32_t node = __shfl_sync(0xffffffffu, val.node, 0);
            if (node < 0) break;
            if constexpr (Layout::kPacked) {
                int32_t row = __shfl_sync(0xffffffffu, val.row, 0);
                if (row < 0) continue;  // outside the sample: no adjacency
                const int2 *src = L.nbr + static_cast<int64_t>(row) * n_nb;
                int2 e0 = __ldg(src + lane);
                if (__shfl_sync(0xffffffffu, e0.x, 0) == kEmptyRowTag) continue;
                v0 = e0.x; r0 = e0.y;
                if (chunks > 1) { int2 e1 = __ldg(src + 32 + lane); v1 = e1.x; r1 = e1.y; }
            } else {
                int64_t lo = 0, hi = 0;
                if (lane == 0) { lo = __ldg(L.indptr + node); hi = __ldg(L.indptr + node + 1); }
                lo = __shfl_sync(0xffffffffu, lo, 0);
                hi = __shfl_sync(0xffffffffu, hi, 0);
                if (lo == hi) continue;
                if (lo + lane < hi) v0 = static_cast<int32_t>(__ldg(L.indices + lo + lane));
                if (chunks > 1 && lo + 32 + lane < hi)
                    v1 = static_cast<int32_t>(__ldg(L.indices + lo + 32 + lane));
            }
            expanding = true;
            break;
        }
        if (expanding) ++n_expand;

        // bloom test-and-set, beams in order (token over named barriers 1..3)
        if (w > 0) named_sync(w, 64);
        bool seen0 = bloom_visit(bloom, v0, lane);
        bool seen1 = true;
        if (chunks > 1) seen1 = bloom_visit(bloom, v1, lane);
        if (w < kBeams - 1) named_arrive(w + 1, 64);

        // compaction in slot order (:151-171)
        uint32_t m0 = __ballot_sync(0xffffffffu, !seen0);
        uint32_t m1 = __ballot_sync(0xffffffffu, !seen1);
        if (lane == 0) counts[w] = __popc(m0) + __popc(m1);
        __syncthreads();
        int before = 0, n_work = 0;
#pragma unroll
        for (int i = 0; i < kBeams; ++i) {
            int c = counts[i];
            if (i < w) before += c;
            n_work += c;
        }
        const uint32_t lt = (1u << lane) - 1u;
        if (!seen0) slots[before + __popc(m0 & lt)] = make_int2(v0, r0);
        if (!seen1) slots[before + __popc(m0) + __popc(m1 & lt)] = make_int2(v1, r1);
        __syncthreads();
        if (n_work < kTeamsPerWarp) break;  // :182-184, uniform over the CTA

        // distances and heap inserts (:187-224): survivor j -> beam (j/4) mod 4,
        // team j mod 4; a beam inserts its survivors in ascending j
        const int team = lane >> 3, t8 = lane & 7;
        for (int j0 = w * kTeamsPerWarp; j0 < n_work; j0 += kBeams * kTeamsPerWarp) {
            int j = j0 + team;
            bool pred = j < n_work;
            int2 s = pred ? slots[j] : make_int2(-1, -1);
            int64_t row;
            if constexpr (Layout::kPacked) row = s.y;
            else row = pred ? __ldg(L.mapping + s.x) : -1;
            pred = pred && row >= 0;
            float dist = team_distance(L.storage + row * d, q_s, d, t8, pred);
#pragma unroll
            for (int i = 0; i < kTeamsPerWarp; ++i) {
                float di = __shfl_sync(0xffffffffu, dist, i * kTeam);
                int32_t ni = __shfl_sync(0xffffffffu, s.x, i * kTeam);
                int32_t ri = __shfl_sync(0xffffffffu, static_cast<int32_t>(row), i * kTeam);
                int pi = __shfl_sync(0xffffffffu, static_cast<int>(pred), i * kTeam);
                if (lane == 0 && pi) {
                    heap_replace(okey, oval, H, di, OpenVal{ni, ri});
                    heap_pushpop(rkey, rid, H, -di, ni);
                    ++n_eval;
                }
            }
        }
    }

    // ---- store (:230-245): per beam worst -> best ----------------------------
    if (lane == 0) {
        float key;
        int32_t id;
        for (int i = ef; i < H; ++i) heap_pop(rkey, rid, H, -1, key, id);
        int64_t *oI = out_I + (b * kBeams + w) * ef;
        float *oD = out_D + (b * kBeams + w) * ef;
        for (int i = 0; i < ef; ++i) {
            heap_pop(rkey, rid, H, -1, key, id);
            oI[i] = id;
            oD[i] = -key;
        }
    }
    if (stats != nullptr) {
        __syncthreads();
        int bits = 0;
        for (int i = threadIdx.x; i < kBloomWords; i += kThreads) bits += __popc(bloom[i]);
        for (int off = 16; off > 0; off >>= 1) bits += __shfl_down_sync(0xffffffffu, bits, off);
        if (lane == 0) {
            atomicAdd(&stat_s[1], n_expand);
            atomicAdd(&stat_s[2], n_eval);
            atomicAdd(&stat_s[3], bits);
            if (w == 0) stat_s[0] = n_rounds;
        }
        __syncthreads();
        if (threadIdx.x < 4) stats[b * 4 + threadIdx.x] = stat_s[threadIdx.x];
    }
}

template <class Layout>
static int launch(Layout L, int64_t *out_I, float *out_D, const float *query, int64_t ldq,
                  const int64_t *init_I, const float *init_D, int64_t batch, int d, int n_nb,
                  int n_init, int ef, int32_t *stats, cudaStream_t stream) {
    if (batch == 0) return PA_OK;
    dim3 grid(static_cast<unsigned>(batch)), block(kThreads);
    size_t dyn = sizeof(float) * d;
#define PA_LAUNCH(HS)                                                                    \
    traverse_kernel<HS, Layout><<<grid, block, dyn, stream>>>(L, out_I, out_D, query,   \
                                                              init_I, init_D, d, ldq,   \
                                                              n_nb, n_init, ef, stats)
    switch (pa_heap_size_for(ef)) {
        case 32: PA_LAUNCH(32); break;
        case 64: PA_LAUNCH(64); break;
        case 128: PA_LAUNCH(128); break;
        default: PA_LAUNCH(256); break;
    }
#undef PA_LAUNCH
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

static int check_common(const void *out_I, const void *out_D, const float *storage,
                        const float *query, const void *init_I, const void *init_D,
                        int64_t batch, int64_t n_nodes, int d, int n_nb, int n_init, int ef) {
    PA_REQUIRE(batch >= 0 && batch <= 0x7fffffff, "batch out of range");
    PA_REQUIRE(pa_heap_size_for(ef) > 0, "ef_search must be in (0, 2048]");
    PA_REQUIRE(n_nb > 0 && n_nb % 32 == 0, "n_neighbors must be a multiple of 32");
    PA_REQUIRE(kBeams * n_nb <= kMaxSlots, "4 * n_neighbors must not exceed 256");
    PA_REQUIRE(d > 0 && d % 4 == 0, "d_model must be a positive multiple of 4");
    PA_REQUIRE(d <= 8192, "d_model too large for the shared-memory query");
    PA_REQUIRE(n_init >= 0, "n_initials must not be negative");
    PA_REQUIRE(n_nodes >= 0 && n_nodes < 0x7fffffff, "node ids must fit int32");
    if (batch == 0) return PA_OK;
    PA_REQUIRE(out_I && out_D && storage && query, "null pointer");
    PA_REQUIRE(n_init == 0 || (init_I && init_D), "null entry pointer");
    PA_REQUIRE(aligned16(storage) && aligned16(query), "storage / query must be 16-byte aligned");
    return PA_OK;
}

int traverse_packed_launch(int64_t *output_I, float *output_D, const int32_t *packed_nbr,
                           const int32_t *row_of, const float *storage, const float *query,
                           int64_t ldq, const int64_t *initial_I, const float *initial_D,
                           int64_t batch, int64_t n_nodes, int64_t n_storage, int d_model,
                           int n_neighbors, int n_initials, int ef_search, int32_t *stats,
                           cudaStream_t stream) {
    (void)n_storage;
    int rc = check_common(output_I, output_D, storage, query, initial_I, initial_D, batch, n_nodes,
                          d_model, n_neighbors, n_initials, ef_search);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(packed_nbr && row_of, "null packed-index pointer");
    PA_REQUIRE((reinterpret_cast<uintptr_t>(packed_nbr) & 7u) == 0,
               "packed_nbr must be 8-byte aligned");
    PA_REQUIRE(ldq >= d_model && ldq % 4 == 0, "query row stride must be a multiple of 4");
    PackedLayout L{reinterpret_cast<const int2 *>(packed_nbr), row_of, storage, n_nodes};
    return launch(L, output_I, output_D, query, ldq, initial_I, initial_D, batch, d_model,
                  n_neighbors, n_initials, ef_search, stats, stream);
}

}  // namespace pa

extern "C" int pa_heap_size_for(int ef) {
    if (ef <= 0 || ef > 2048) return -1;
    if (ef <= 32) return 32;
    if (ef <= 64) return 64;
    if (ef <= 128) return 128;
    return 256;
}

extern "C" int pa_traverse_csr(int64_t *output_I, float *output_D, const int64_t *indptr,
                               const int64_t *indices, const int64_t *mapping,
                               const float *storage, const float *query,
                               const int64_t *initial_I, const float *initial_D, int64_t batch,
                               int64_t n_nodes, int64_t n_storage, int d_model, int n_neighbors,
                               int n_initials, int ef_search, int32_t *stats, void *stream) {
    (void)n_storage;
    int rc = pa::check_common(output_I, output_D, storage, query, initial_I, initial_D, batch,
                              n_nodes, d_model, n_neighbors, n_initials, ef_search);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(indptr && indices && mapping, "null graph pointer");
    pa::CsrLayout L{indptr, indices, mapping, storage, n_nodes};
    return pa::launch(L, output_I, output_D, query, d_model, initial_I, initial_D, batch,
                      d_model, n_neighbors, n_initials, ef_search, stats,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int pa_traverse_packed(int64_t *output_I, float *output_D, const int32_t *packed_nbr,
                                  const int32_t *row_of, const float *storage,
                                  const float *query, const int64_t *initial_I,
                                  const float *initial_D, int64_t batch, int64_t n_nodes,
                                  int64_t n_storage, int d_model, int n_neighbors,
                                  int n_initials, int ef_search, int32_t *stats, void *stream) {
    return pa::traverse_packed_launch(output_I, output_D, packed_nbr, row_of, storage, query,
                                      d_model, initial_I, initial_D, batch, n_nodes, n_storage,
                                      d_model, n_neighbors, n_initials, ef_search, stats,
                                      static_cast<cudaStream_t>(stream));
}

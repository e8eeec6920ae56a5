/*
 * pilot_oracle.c -- CPU restatement of the PilotANN GPU search stage.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels of
 * this repository; it is never part of the product path.  Only the tests, the
 * smoke check and the CPU-baseline leg of the benchmark may load it.
 *
 * Every function restates one piece of the upstream project (paths are relative
 * to the upstream repository root):
 *
 *   po_fnv1a_32 / po_bloom_positions   extension/inc/bloom.cuh:9-16,
 *                                      extension/traverse_cuda.cu:60-74
 *   po_heap_pop / _replace / _pushpop  extension/inc/heapq.cuh:13-87
 *   po_reduced_distance                extension/traverse_cuda.cu:18-43
 *   po_traverse                        extension/traverse_cuda.cu:45-246, 249-315
 *   po_route                           extension/routing_cuda.cu:10-66, 70-113 and
 *                                      pilot_ann/layers/entry.py:81-88
 *   po_project                         pilot_ann/layers/staged.py:198
 *   po_search_cpu / po_refine          extension/traverse_cpu.cpp:12-163, 167-257,
 *                                      261-369 (the CPU consumer of the handoff)
 *   po_refine_ex                       the same two stages with the summation
 *                                      order of the GPU refinement kernel
 *                                      (po_warp_distance) instead of the AVX2 one,
 *                                      so that kernel can be compared bit for bit;
 *                                      stage 2 alone or stages 2 + 3
 *
 * The upstream GPU kernel is racy (four warps race on the bloom filter, all 32
 * lanes of a warp redundantly run the heap code).  This restatement fixes ONE
 * legal interleaving of it, and the CUDA kernels of this repository implement
 * the very same one, so that the two can be compared bit for bit:
 *
 *   - the bloom filter is cleared before the first use;
 *   - within a round the neighbour slots are visited beam 0 -> 3, and within a
 *     beam in chunks of 32 lanes; a chunk runs the four hash steps in lock step
 *     (step-major), and within one step lanes that touch the same bit are
 *     served in ascending lane order;
 *   - heap code runs once per warp (the 32 redundant copies write equal values).
 *
 * Parity status: pinned.  The heap routines are compared against the upstream
 * heapq.cuh through oracle/_ref (random operation traces), po_search_cpu /
 * po_refine against the upstream traverse_cpu / traverse_refine, and
 * po_traverse / po_route against the upstream CUDA kernels when a GPU is
 * present (tests/test_oracle_pin.py, tests/test_parity_reference_gpu.py).
 *
 * Floating point: compile with -ffp-contract=off; every fused multiply-add is
 * written as fmaf() so that the rounding sequence is the one the CUDA kernels
 * spell out with __fmaf_rn / __fadd_rn.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PO_BEAMS 4
#define PO_BLOOM_BITS 32768u
#define PO_BLOOM_WORDS (PO_BLOOM_BITS / 32u)
#define PO_FNV_STEPS 4
#define PO_FNV_PRIME 0x01000193u
#define PO_FNV_OFFSET 0x811c9dc5u
#define PO_MAX_SLOTS 256 /* BUFFER_SIZE, traverse_cuda.cu:14 */

/* ------------------------------------------------------------------ bloom */

/* bloom.cuh:9-16 -- note that the whole shifted word is xor-ed in, not a byte */
uint32_t po_fnv1a_32(uint32_t x, uint32_t offset) {
    uint32_t h = offset;
    for (int i = 0; i < 4; i++) {
        h ^= x >> (8 * i);
        h *= PO_FNV_PRIME;
    }
    return h;
}

/* traverse_cuda.cu:65-69 -- the four chained bit positions of one node id */
void po_bloom_positions(int64_t node, uint32_t pos[PO_FNV_STEPS]) {
    uint32_t h = PO_FNV_OFFSET;
    for (int s = 0; s < PO_FNV_STEPS; s++) {
        h = po_fnv1a_32((uint32_t)node, h);
        pos[s] = h % PO_BLOOM_BITS;
    }
}

static inline int bloom_test_and_set(uint32_t *bloom, uint32_t pos) {
    uint32_t w = pos >> 5, b = pos & 31u;
    int old = (int)((bloom[w] >> b) & 1u);
    bloom[w] |= 1u << b;
    return old;
}

/* ------------------------------------------------------------------- heaps */

/* heapq.cuh:13-29 (named __heapify_up upstream; it sifts the root down) */
static void sift_root_down(float *keys, int64_t *values, int hsize) {
    for (int cursor = 0, child = 1; child < hsize;
         cursor = child, child = 2 * cursor + 1) {
        int right = child + 1;
        if (right < hsize && keys[right] < keys[child]) child = right;
        if (keys[cursor] <= keys[child]) break;
        float tk = keys[cursor]; keys[cursor] = keys[child]; keys[child] = tk;
        int64_t tv = values[cursor]; values[cursor] = values[child]; values[child] = tv;
    }
}

/* heapq.cuh:38-45 */
void po_heap_pop(float *keys, int64_t *values, int hsize, float *out_key,
                 int64_t *out_value) {
    *out_key = keys[0];
    *out_value = values[0];
    keys[0] = INFINITY;
    values[0] = -1;
    sift_root_down(keys, values, hsize);
}

/* heapq.cuh:47-77 -- walk to a leaf along the larger child, replace it if the
 * new key is smaller, sift up */
void po_heap_replace(float *keys, int64_t *values, int hsize, float k, int64_t v) {
    int cursor = 0;
    for (int child = 1; child < hsize; cursor = child, child = 2 * cursor + 1) {
        int right = child + 1;
        if (right < hsize && keys[right] > keys[child]) child = right;
    }
    if (k >= keys[cursor]) return;
    keys[cursor] = k;
    values[cursor] = v;
    while (cursor > 0) {
        int parent = (cursor - 1) / 2;
        if (keys[parent] <= keys[cursor]) break;
        float tk = keys[cursor]; keys[cursor] = keys[parent]; keys[parent] = tk;
        int64_t tv = values[cursor]; values[cursor] = values[parent]; values[parent] = tv;
        cursor = parent;
    }
}

/* heapq.cuh:79-87 */
void po_heap_pushpop(float *keys, int64_t *values, int hsize, float k, int64_t v) {
    if (k <= keys[0]) return;
    keys[0] = k;
    values[0] = v;
    sift_root_down(keys, values, hsize);
}

/* ---------------------------------------------------------------- distance */

/* traverse_cuda.cu:18-43.  Eight lanes; lane t owns floats [32m+4t, 32m+4t+4);
 * per stripe: acc += fma(dx,dx,dy*dy); acc += fma(dz,dz,dw*dw); then the
 * width-8 shuffle tree with offsets 4, 2, 1. */
float po_reduced_distance(const float *row, const float *query, int d) {
    float lane[8];
    for (int t = 0; t < 8; t++) {
        float acc = 0.0f;
        for (int off = 0; off < d; off += 32) {
            int i = off + 4 * t;
            if (i < d) {
                float dx = query[i] - row[i], dy = query[i + 1] - row[i + 1];
                float dz = query[i + 2] - row[i + 2], dw = query[i + 3] - row[i + 3];
                acc = acc + fmaf(dx, dx, dy * dy);
                acc = acc + fmaf(dz, dz, dw * dw);
            }
        }
        lane[t] = acc;
    }
    for (int off = 4; off > 0; off /= 2)
        for (int t = 0; t < off; t++) lane[t] = lane[t] + lane[t + off];
    return lane[0];
}

/* --------------------------------------------------------------- traversal */

static int heap_size_for(int ef) { /* traverse_cuda.cu:302-315 */
    if (ef <= 32) return 32;
    if (ef <= 64) return 64;
    if (ef <= 128) return 128;
    if (ef <= 2048) return 256;
    return -1;
}

int po_heap_size_for(int ef) { return heap_size_for(ef); }

/* One query.  stats (optional, 4 ints): rounds entered, nodes expanded (E),
 * distance evaluations (C), bloom bits set at the end. */
static void traverse_one(int64_t *out_I, float *out_D, const int64_t *indptr,
                         const int64_t *indices, const int64_t *mapping,
                         const float *storage, const float *query,
                         const int64_t *init_I, const float *init_D, int d,
                         int n_nb, int n_init, int ef, int H, int32_t *stats) {
    uint32_t bloom[PO_BLOOM_WORDS];
    memset(bloom, 0, sizeof bloom);
    float *buf_D = malloc(sizeof(float) * PO_BEAMS * H * 2);
    int64_t *buf_I = malloc(sizeof(int64_t) * PO_BEAMS * H * 2);
    float *open_D = buf_D + PO_BEAMS * H;
    int64_t *open_I = buf_I + PO_BEAMS * H;
    for (int i = 0; i < PO_BEAMS * H; i++) {
        buf_D[i] = -INFINITY; buf_I[i] = -1;
        open_D[i] = INFINITY; open_I[i] = -1;
    }
    int32_t n_rounds = 0, n_expand = 0, n_eval = 0;

    /* init, traverse_cuda.cu:96-111: entry i goes to beam i mod 4 */
    for (int i = 0; i < n_init; i++) {
        int w = i % PO_BEAMS;
        int64_t node = init_I[i];
        float dist = init_D[i];
        if (node < 0 || dist >= -buf_D[w * H]) continue;
        po_heap_replace(open_D + w * H, open_I + w * H, H, dist, node);
        po_heap_pushpop(buf_D + w * H, buf_I + w * H, H, -dist, node);
        uint32_t pos[PO_FNV_STEPS];
        po_bloom_positions(node, pos);
        for (int s = 0; s < PO_FNV_STEPS; s++) bloom_test_and_set(bloom, pos[s]);
    }

    int64_t slots[PO_MAX_SLOTS];
    for (int step = 0; step < ef; step++) {
        n_rounds++;
        /* pop, traverse_cuda.cu:118-134 */
        int64_t u[PO_BEAMS];
        for (int w = 0; w < PO_BEAMS; w++) {
            u[w] = -1;
            for (;;) {
                float key; int64_t val;
                po_heap_pop(open_D + w * H, open_I + w * H, H, &key, &val);
                if (val < 0) break;
                if (key >= -buf_D[w * H]) break;
                if (indptr[val] == indptr[val + 1]) continue;
                u[w] = val;
                break;
            }
            if (u[w] >= 0) n_expand++;
        }
        /* expand, traverse_cuda.cu:137-146, in the fixed schedule */
        for (int w = 0; w < PO_BEAMS; w++) {
            for (int base = 0; base < n_nb; base += 32) {
                int64_t v[32]; int valid[32], found[32]; uint32_t pos[32][PO_FNV_STEPS];
                for (int lane = 0; lane < 32; lane++) {
                    int i = base + lane;
                    valid[lane] = 0; v[lane] = -1; found[lane] = 1;
                    if (i < n_nb && u[w] >= 0 && indptr[u[w]] + i < indptr[u[w] + 1]) {
                        v[lane] = indices[indptr[u[w]] + i];
                        if (v[lane] >= 0) {
                            valid[lane] = 1;
                            po_bloom_positions(v[lane], pos[lane]);
                        }
                    }
                }
                for (int s = 0; s < PO_FNV_STEPS; s++)
                    for (int lane = 0; lane < 32; lane++)
                        if (valid[lane])
                            found[lane] &= bloom_test_and_set(bloom, pos[lane][s]);
                for (int lane = 0; lane < 32 && base + lane < n_nb; lane++)
                    slots[w * n_nb + base + lane] =
                        (valid[lane] && !found[lane]) ? v[lane] : -1;
            }
        }
        /* compact, traverse_cuda.cu:151-171 */
        int n_work = 0;
        for (int i = 0; i < PO_BEAMS * n_nb; i++)
            if (slots[i] >= 0) slots[n_work++] = slots[i];
        if (n_work < 4) break; /* traverse_cuda.cu:182-184 */
        /* distances + inserts, traverse_cuda.cu:187-224: survivor j belongs to
         * beam (j / 4) mod 4; a beam inserts its survivors in ascending j */
        for (int j = 0; j < n_work; j++) {
            int w = (j / 4) % PO_BEAMS;
            int64_t node = slots[j];
            int64_t loc = mapping[node];
            if (loc < 0) continue;
            float dist = po_reduced_distance(storage + loc * (int64_t)d, query, d);
            n_eval++;
            po_heap_replace(open_D + w * H, open_I + w * H, H, dist, node);
            po_heap_pushpop(buf_D + w * H, buf_I + w * H, H, -dist, node);
        }
    }

    /* store, traverse_cuda.cu:230-245: worst -> best per beam */
    for (int w = 0; w < PO_BEAMS; w++) {
        float key; int64_t val;
        for (int i = ef; i < H; i++)
            po_heap_pop(buf_D + w * H, buf_I + w * H, H, &key, &val);
        for (int i = 0; i < ef; i++) {
            po_heap_pop(buf_D + w * H, buf_I + w * H, H, &key, &val);
            out_I[w * ef + i] = val;
            out_D[w * ef + i] = -key;
        }
    }
    if (stats) {
        int bits = 0;
        for (unsigned i = 0; i < PO_BLOOM_WORDS; i++) bits += __builtin_popcount(bloom[i]);
        stats[0] = n_rounds; stats[1] = n_expand; stats[2] = n_eval; stats[3] = bits;
    }
    free(buf_D);
    free(buf_I);
}

/* Reference-layout traversal of a batch.  Shapes as extension/entry.cpp:32-38:
 * out_* [B,4,ef], indptr [n_nodes+1], indices [*], mapping [n_nodes],
 * storage [n_storage,d], query [B,d], init_* [B,n_init].  Returns 0, or -1 for
 * arguments the upstream launcher rejects (traverse_cuda.cu:280-281, :313). */
int po_traverse(int64_t *out_I, float *out_D, const int64_t *indptr,
                const int64_t *indices, const int64_t *mapping,
                const float *storage, const float *query, const int64_t *init_I,
                const float *init_D, int64_t batch, int d, int n_nb, int n_init,
                int ef, int32_t *stats) {
    int H = heap_size_for(ef);
    if (H < 0 || n_nb % 32 != 0 || PO_BEAMS * n_nb > PO_MAX_SLOTS || d % 4 != 0)
        return -1;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t b = 0; b < batch; b++)
        traverse_one(out_I + b * PO_BEAMS * ef, out_D + b * PO_BEAMS * ef, indptr,
                     indices, mapping, storage, query + b * d, init_I + b * n_init,
                     init_D + b * n_init, d, n_nb, n_init, ef, H,
                     stats ? stats + 4 * b : NULL);
    return 0;
}

/* ----------------------------------------------------------------- routing */

/* routing_cuda.cu:93-95 picks the router with argmin(cdist(query, routers)).
 * Here the squared distance is accumulated in double precision, which orders
 * the routers as exact arithmetic on the float inputs would (ties -> lowest
 * index).  routing_cuda.cu:10-66 then accumulates, for the chosen router's
 * leaves, sum_k (q_k - p_k)^2 in fp32: per 32-wide k tile a running
 * r = fma(q - p, q - p, r) from 0, the tile sums added in tile order to a total
 * that starts at 0.  entry.py:86-88 gathers the leaf ids of the chosen router. */
int po_route(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
             const float *route_vectors, const int64_t *entry_nodes,
             const float *entry_vectors, int64_t batch, int d, int n_routers,
             int n_leaves) {
    if (n_leaves % 32 != 0) return -1; /* routing_cuda.cu:90 */
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < batch; b++) {
        const float *q = query + b * d;
        int best = 0;
        double best_d = INFINITY;
        for (int r = 0; r < n_routers; r++) {
            const float *p = route_vectors + (int64_t)r * d;
            double acc = 0.0;
            for (int k = 0; k < d; k++) {
                double diff = (double)q[k] - (double)p[k];
                acc += diff * diff;
            }
            if (acc < best_d) { best_d = acc; best = r; }
        }
        router[b] = best;
        for (int l = 0; l < n_leaves; l++) {
            const float *p = entry_vectors + ((int64_t)best * n_leaves + l) * d;
            float total = 0.0f;
            for (int k0 = 0; k0 < d; k0 += 32) {
                float r = 0.0f;
                for (int k = k0; k < k0 + 32; k++) {
                    /* out-of-range columns are staged as zeros upstream */
                    float diff = (k < d) ? q[k] - p[k] : 0.0f;
                    r = fmaf(diff, diff, r);
                }
                total = total + r;
            }
            leaf_D[b * n_leaves + l] = total;
            if (leaf_I) leaf_I[b * n_leaves + l] = entry_nodes[(int64_t)best * n_leaves + l];
        }
    }
    return 0;
}

/* -------------------------------------------------------------- projection */

/* staged.py:198: rotated = query @ VT.T, i.e. out[b,j] = sum_k q[b,k] * VT[j,k].
 * Accumulated in double precision and rounded once; the tensor-core kernel is
 * compared within a tolerance.  Only the first d_out rows of VT are used. */
void po_project(float *out, const float *query, const float *VT, int64_t batch,
                int d, int d_out) {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < batch; b++)
        for (int j = 0; j < d_out; j++) {
            double acc = 0.0;
            for (int k = 0; k < d; k++)
                acc += (double)query[b * d + k] * (double)VT[(int64_t)j * d + k];
            out[b * d_out + j] = (float)acc;
        }
}

/* --------------------------------------------- CPU consumer of the handoff */

/* distance.h:31-58: eight running sums (one per AVX lane), lane sums added in
 * lane order.  -ffast-math upstream may reorder the final adds; results are
 * compared within a tolerance, ids exactly except on such ties. */
static float dist_avx_order(const float *q, const float *x, int d, int offset) {
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int o = offset; o < d; o += 8)
        for (int k = 0; k < 8; k++) {
            float t = q[o + k] - x[o + k];
            lane[k] = fmaf(t, t, lane[k]);
        }
    float r = 0.0f;
    for (int k = 0; k < 8; k++) r += lane[k];
    return r;
}

/* traverse_cpu.cpp:12-163.  `visited` is the epoch-marker array of
 * bitmask.hpp:12-45 (int32 per node, value == marker means visited). */
/* Summation order of the GPU refinement kernel: 32 lanes, lane t owns floats
 * [offset + 128m + 4t, +4); per stripe acc += fma(dx,dx,dy*dy); acc +=
 * fma(dz,dz,dw*dw) in ascending m; then the butterfly 16, 8, 4, 2, 1 (lane 0 of a
 * shuffle-xor butterfly adds in exactly this order, and every lane ends with the
 * same bits because the additions commute). */
float po_warp_distance(const float *q, const float *x, int d, int offset) {
    float lane[32];
    for (int t = 0; t < 32; t++) {
        float acc = 0.0f;
        for (int o = offset + 4 * t; o < d; o += 128) {
            float dx = q[o] - x[o], dy = q[o + 1] - x[o + 1];
            float dz = q[o + 2] - x[o + 2], dw = q[o + 3] - x[o + 3];
            acc = acc + fmaf(dx, dx, dy * dy);
            acc = acc + fmaf(dz, dz, dw * dw);
        }
        lane[t] = acc;
    }
    for (int off = 16; off > 0; off /= 2)
        for (int t = 0; t < off; t++) lane[t] = lane[t] + lane[t + off];
    return lane[0];
}

static float full_dist(const float *q, const float *x, int d, int offset, int dist_mode) {
    return dist_mode ? po_warp_distance(q, x, d, offset) : dist_avx_order(q, x, d, offset);
}

/* traverse_cpu.cpp:12-163.  `visited` is the epoch-marker array of
 * bitmask.hpp:12-45 (int32 per node, value == marker means visited).
 * dist_mode 0: AVX2 summation order (the one pinned to upstream); 1: the GPU
 * kernel's.  stats (optional, 2 ints): nodes expanded, distance evaluations. */
static void search_cpu_one(int64_t *out_I, float *out_D, int32_t *visited,
                           int64_t *init_I, float *init_D, const int64_t *indptr,
                           const int64_t *indices, const float *storage,
                           const float *query, int d, int d_principle, int n_init,
                           int ef, int k, int H, int32_t marker, int max_iter,
                           int dist_mode, int32_t *stats) {
    float *buf_D = malloc(sizeof(float) * 3 * H);
    int64_t *buf_I = malloc(sizeof(int64_t) * 3 * H);
    float *open_D = buf_D + H;
    int64_t *open_I = buf_I + H;
    int32_t n_expand = 0, n_eval = 0;
    if (d_principle < d) /* :41-62 residual over the trailing dims, in place */
        for (int i = 0; i < n_init; i++)
            if (init_I[i] >= 0)
                init_D[i] += full_dist(query, storage + init_I[i] * (int64_t)d, d,
                                       d_principle, dist_mode);
    for (int i = 0; i < H; i++) { buf_D[i] = -INFINITY; buf_I[i] = -1; }
    for (int i = 0; i < 2 * H; i++) { open_D[i] = INFINITY; open_I[i] = -1; }
    for (int i = 0; i < n_init; i++) { /* :69-79 */
        int64_t u = init_I[i];
        if (u < 0) continue;
        visited[u] = marker;
        po_heap_replace(open_D, open_I, 2 * H, init_D[i], u);
    }
    if (max_iter > 2 * ef) max_iter = 2 * ef; /* :82 */
    for (int step = 0; step < max_iter; step++) {
        float key; int64_t u;
        po_heap_pop(open_D, open_I, 2 * H, &key, &u);
        if (u < 0 || key >= -buf_D[0]) break;
        n_expand++;
        for (int64_t i = indptr[u]; i < indptr[u + 1]; i++) { /* :105-135 */
            int64_t v = indices[i];
            if (v < 0) break;
            if (visited[v] == -1 || visited[v] == marker) continue;
            visited[v] = marker;
            float dist = full_dist(query, storage + v * (int64_t)d, d, 0, dist_mode);
            n_eval++;
            if (dist >= -buf_D[0]) continue; /* :27-29 */
            po_heap_pushpop(buf_D, buf_I, H, -dist, v);
            po_heap_replace(open_D, open_I, 2 * H, dist, v);
        }
    }
    for (int i = 0; i < n_init; i++) /* :139-148 */
        if (init_I[i] >= 0) po_heap_pushpop(buf_D, buf_I, H, -init_D[i], init_I[i]);
    float key; int64_t val;
    for (int i = k; i < H; i++) po_heap_pop(buf_D, buf_I, H, &key, &val);
    for (int i = 0; i < k; i++) { /* :156-162: ascending */
        po_heap_pop(buf_D, buf_I, H, &key, &val);
        out_I[k - i - 1] = val;
        out_D[k - i - 1] = -key;
    }
    if (stats) { stats[0] = n_expand; stats[1] = n_eval; }
    free(buf_D);
    free(buf_I);
}

static int cpu_heap_size_for(int ef) { /* traverse_cpu.cpp:228-254 */
    static const int sizes[] = {16, 32, 48, 64, 96, 128, 192, 256, 384, 512, 1024, 2048};
    for (unsigned i = 0; i < sizeof sizes / sizeof sizes[0]; i++)
        if (ef <= sizes[i]) return sizes[i];
    return -1;
}

/* traverse_cpu.cpp:167-257: best-first search on the full graph. init_* are
 * read only here (d_principle == d).  Returns 0 or -1. */
int po_search_cpu(int64_t *out_I, float *out_D, int64_t *init_I, float *init_D,
                  const int64_t *indptr, const int64_t *indices, const float *storage,
                  const float *query, int64_t batch, int64_t n_storage, int d,
                  int n_init, int k, int ef) {
    int H = cpu_heap_size_for(ef);
    if (H < 0) return -1;
#pragma omp parallel
    {
        int32_t *visited = calloc((size_t)n_storage, sizeof(int32_t));
        int32_t marker = 0;
#pragma omp for schedule(guided)
        for (int64_t b = 0; b < batch; b++) {
            marker++;
            search_cpu_one(out_I + b * k, out_D + b * k, visited, init_I + b * n_init,
                           init_D + b * n_init, indptr, indices, storage,
                           query + b * d, d, d, n_init, ef, k, H, marker, 1024, 0, NULL);
        }
        free(visited);
    }
    return 0;
}

int po_cpu_heap_size_for(int ef) { return cpu_heap_size_for(ef); }

/* traverse_cpu.cpp:261-369: stage 2 (subgraph, residual fix-up, two expansion
 * steps, result written back into the handoff buffer) then stage 3 (full
 * graph).  buffer_* [B,n_buf] is the handoff, read and overwritten.
 * dist_mode: see search_cpu_one.  stages: 2 = stage 2 only (out_* untouched),
 * 3 = both.  stats: NULL or int32 [B,4] = stage-2 expansions, stage-2
 * evaluations, stage-3 expansions, stage-3 evaluations. */
int po_refine_ex(int64_t *out_I, float *out_D, int64_t *buffer_I, float *buffer_D,
                 const int64_t *sub_indptr, const int64_t *sub_indices,
                 const int64_t *full_indptr, const int64_t *full_indices,
                 const float *storage, const float *query, int64_t batch,
                 int64_t n_storage, int d, int d_principle, int n_buf, int k, int ef,
                 int dist_mode, int stages, int32_t *stats) {
    int H = cpu_heap_size_for(ef);
    if (H < 0) return -1;
#pragma omp parallel
    {
        int32_t *visited = calloc((size_t)n_storage, sizeof(int32_t));
        int32_t marker = 0;
#pragma omp for schedule(guided)
        for (int64_t b = 0; b < batch; b++) {
            marker++;
            int64_t *bI = buffer_I + b * n_buf;
            float *bD = buffer_D + b * n_buf;
            int32_t st[4] = {0, 0, 0, 0};
            /* the stage-2 call reads and writes the same rows (pipeline_cpu.cpp:
             * 110-114 passes one tensor as both); snapshot the inputs first so
             * that the write-back cannot disturb them */
            int64_t *tI = malloc(sizeof(int64_t) * n_buf);
            float *tD = malloc(sizeof(float) * n_buf);
            memcpy(tI, bI, sizeof(int64_t) * n_buf);
            memcpy(tD, bD, sizeof(float) * n_buf);
            search_cpu_one(bI, bD, visited, tI, tD, sub_indptr, sub_indices, storage,
                           query + b * d, d, d_principle, n_buf, ef, n_buf, H, marker, 2,
                           dist_mode, st);
            if (stages >= 3)
                search_cpu_one(out_I + b * k, out_D + b * k, visited, bI, bD, full_indptr,
                               full_indices, storage, query + b * d, d, d, n_buf, ef, k, H,
                               marker, 1024, dist_mode, st + 2);
            if (stats) memcpy(stats + 4 * b, st, sizeof st);
            free(tI);
            free(tD);
        }
        free(visited);
    }
    return 0;
}

int po_refine(int64_t *out_I, float *out_D, int64_t *buffer_I, float *buffer_D,
              const int64_t *sub_indptr, const int64_t *sub_indices,
              const int64_t *full_indptr, const int64_t *full_indices,
              const float *storage, const float *query, int64_t batch,
              int64_t n_storage, int d, int d_principle, int n_buf, int k, int ef) {
    return po_refine_ex(out_I, out_D, buffer_I, buffer_D, sub_indptr, sub_indices, full_indptr,
                        full_indices, storage, query, batch, n_storage, d, d_principle, n_buf, k,
                        ef, 0, 3, NULL);
}

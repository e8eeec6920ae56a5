// Refinement of the candidate handoff on the GPU: the two stages upstream runs on
// the CPU in `traverse_refine` (extension/traverse_cpu.cpp:261-369), each of them
// one call of `traverse_cpu_kernel` (:12-163):
//
//   stage 2  the [batch, 4 * ef] candidates of the reduced-space traversal get
//            their distances completed over dims d_principle .. d_model (:41-62),
//            seed a best-first search on the SUB-graph that is cut off after
//            REFINE_STEP = 2 expansions (:64-136), and the best H of candidates
//            and newly found nodes are written back, ascending, behind (-1, -inf)
//            pads (:138-162);
//   stage 3  the same search, seeded with the stage-2 result, on the FULL graph
//            with full-dimension distances, up to 2 * ef expansions, top-k out.
//
// The candidates are consumed where the traversal left them, in HBM; nothing of
// the handoff crosses PCIe.  One CTA of five warps (three for rows of at most 512
// bytes) per query, persistent: CTA i owns slot i of the visited-set pool
// (visited.cu), starts on query i and claims further queries from a counter.
// Warp 0 is the heap warp (it runs upstream's heap routines), the other warps
// gather: adjacency row, visited marks, vector rows, distances.  Three serial
// pieces of upstream's routine -- pushing the seeds into the open heap of the
// two-expansion stage, seeding the full-graph stage, merging seeds and result --
// are computed from their outcome when the keys involved are pairwise different
// (brief_search, the seeding in search_stage, select_sort_output) and run as
// upstream wrote them otherwise.  In the full-graph stage the two sides overlap: the node the next
// pop will return is known as soon as the distances of the current expansion are
// (it is the better of the open heap's root and the best new neighbour -- a new
// key below the root always sifts up to the root, equal keys never pass it), so
// the gather warps start on that node while the heap warp still inserts the
// current expansion's neighbours and pops.  The pop then either confirms the
// node or ends the search (when the best new neighbour is not admitted to the
// heaps the next pop fails the stop test), in which case the speculative marks
// are never looked at again.  The sub-graph stage does not speculate: its marks
// are inherited by the full-graph stage.  Semantics are upstream's, operation
// for operation:
//   * the result heap (H entries) and the open heap (2H entries) are upstream's
//     array heaps with upstream's routines (extension/inc/heapq.cuh:13-87) --
//     heap_replace evicts the leaf reached by walking larger children, not the
//     maximum, so the layout is part of the result; they live in shared memory,
//     stored 1-based as {key, id} pairs so that both children of a node come in
//     one 16-byte load, and are driven by the 32 lanes of the heap warp together
//     (see the routines below);
//   * H follows upstream's CPU dispatch (traverse_cpu.cpp:228-254);
//   * exact visited marks (extension/inc/bitmask.hpp:12-45) shared by the two
//     stages of a query, as upstream shares one marker between them;
//   * neighbours are taken in row order, a row ends at its first negative id.
// Distances: one warp per vector row, lane t owns floats [128m + 4t, +4),
// acc += fma(dx,dx,dy*dy); acc += fma(dz,dz,dw*dw) in ascending m, butterfly
// 16..1.  Upstream's AVX2 order (eight running sums, built with -ffast-math)
// differs from this in the last bits, so results agree with upstream's within a
// relative 1e-5 and with the CPU oracle, which restates this order, bit for bit.
#include "pa_common.cuh"

namespace pa {

// Warp 0 runs the heaps, the other warps gather.  The kernel is compiled for CTAs of
// up to five warps; vector rows of at most 512 bytes are served by two gather warps
// (96 threads), which lets twelve instead of seven queries share an SM -- at those
// sizes the heap warp, not the gather, sets the pace of a query -- or by three when
// the batch leaves room for them (nine queries per SM).
#ifndef PA_REFINE_WIDE_THREADS
#define PA_REFINE_WIDE_THREADS 160
#endif
#ifndef PA_REFINE_NARROW_THREADS
#define PA_REFINE_NARROW_THREADS 96
#endif
#ifndef PA_REFINE_NARROW_DIM
#define PA_REFINE_NARROW_DIM 128
#endif
constexpr int kRefThreads = 160;  // what the kernel is compiled for
constexpr int kRefThreadsWide = PA_REFINE_WIDE_THREADS;
constexpr int kRefThreadsNarrow = PA_REFINE_NARROW_THREADS;
constexpr int kNarrowMaxDim = PA_REFINE_NARROW_DIM;
static_assert(kRefThreadsWide <= kRefThreads && kRefThreadsNarrow <= kRefThreads &&
                  kRefThreadsNarrow >= 64 && kRefThreadsWide % 32 == 0 && kRefThreadsNarrow % 32 == 0,
              "a heap warp plus one to four gather warps");
__host__ __device__ inline int ref_threads_for(int d) {
    return d <= kNarrowMaxDim ? kRefThreadsNarrow : kRefThreadsWide;
}
#ifndef PA_REFINE_MIN_CTAS
#define PA_REFINE_MIN_CTAS 7
#endif
// PA_REFINE_PROFILE (experiments only): 1 = thread 0 (heap warp) accumulates clock
// deltas per phase into stats[b * 24 + 4 ..] and thread 32 (first gather warp) into
// stats[b * 24 + 12 ..]; 2 = thread 32 only.  The stats rows are then 24 ints wide.
// A clock read may still move across a barrier, so a wait can land in the
// neighbouring phase's count; and the heap warp's own clocks slow its heap routines
// several times over while the gather warps run beside it -- read the heap warp's
// cost from mode 2 (how long the gather warps wait for it).
#ifndef PA_REFINE_PROFILE
#define PA_REFINE_PROFILE 0
#endif
#if PA_REFINE_PROFILE
__device__ __forceinline__ long long pinned_clock() {
    long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
    return t;
}
#define PA_TICK(slot) do { if (PA_REFINE_PROFILE == 1 && threadIdx.x == 0) { const long long now__ = pinned_clock(); prof[slot] += static_cast<int>(now__ - prof_t); prof_t = now__; } } while (0)
#define PA_GTICK(slot) do { if (threadIdx.x == 32) { const long long now__ = pinned_clock(); prof[slot] += static_cast<int>(now__ - prof_t); prof_t = now__; } } while (0)
#else
#define PA_TICK(slot) do { } while (0)
#define PA_GTICK(slot) do { } while (0)
#endif
constexpr int kMaxDegree = 64;
constexpr unsigned kAll = 0xffffffffu;

struct RefGraph {
    const int32_t *nbr;     // neighbour ids
    const int32_t *row_of;  // node -> row, or nullptr when the row is the node id
    int64_t row_stride;     // ints between rows
    int elem_stride;        // ints between the ids of a row
    int degree;             // slots per row
};

struct RefineArgs {
    const int64_t *cand_I;  // [batch, n_cand]
    const float *cand_D;
    const float *query;     // [batch, ldq] full rotated queries
    int64_t ldq;
    const float *storage;   // [n_nodes, d] full vectors
    int64_t n_nodes;
    int d, d_p;
    RefGraph sub, full;
    int n_cand, ef, H, k, stages, batch;
    int64_t *out_I;         // stages 2: [batch, n_cand]; stages 3: [batch, k]
    float *out_D;
    uint8_t *marks;         // visited pool: slot s at marks + s * slot_stride
    int32_t *epoch;         // [slots] last marker used by the slot
    unsigned *claim;        // queries handed out beyond each CTA's first, this launch
    int64_t slot_stride;
    int slot_begin;
    int32_t *stats;         // nullptr or [batch, 4]
};

// ---- upstream's heaps, 1-based {key, id} pairs, one warp ------------------------
struct __align__(8) HeapEntry {
    float k;
    int32_t v;
};

// h[1 .. n] is the heap (upstream index c lives at c + 1); h[n + 1] exists and is
// never meaningful: the pair load of the last parent may touch it.  Both children
// of node c sit in one aligned 16-byte pair at h + 2c.
//
// Upstream's routines walk from the root to a leaf, one dependent comparison per
// level.  Here the 32 lanes of the heap warp look at the five levels below the
// current node at once: lane l owns the l-th node of that sub-tree (heap order),
// compares its two children, a ballot collects the 31 decisions, every lane then
// tests with one mask compare whether its own node lies on the path those
// decisions describe, and a second ballot yields the path -- its highest set bit
// is the node five levels down.  Two such steps cover a heap of 1024 entries.  The
// keys along the path are then loaded one per lane and a ballot tells how far the
// moving key travels; the shift of the path is one store per lane.  The heap is
// not touched between the decisions and the stores, so the result is upstream's
// array, entry for entry (checked on the host against the oracle's routines over
// 2 M random operations at sizes 1 .. 4096, odd sizes included).

struct WalkLane {    // what a lane needs to know about its place in a 5-level sub-tree
    int depth, off;  // node = (root << depth) + off
    unsigned care, want;  // on the path iff (decisions & care) == want
};

__device__ __forceinline__ WalkLane walk_lane(int lane) {
    WalkLane L;
    const int r = lane + 1;
    L.depth = 31 - __clz(r);
    L.off = r - (1 << L.depth);
    L.care = L.want = 0;
#pragma unroll
    for (int t = 1; t <= 4; ++t) {
        if (t <= L.depth) {
            const int q = r >> t;  // ancestor; it has to point at (r >> (t - 1))
            L.care |= 1u << (q - 1);
            L.want |= static_cast<unsigned>((r >> (t - 1)) & 1) << (q - 1);
        }
    }
    return L;
}

// Leaf reached from the root by taking the larger (kLarger) or the smaller child
// at every node; the right child wins only if it exists and is strictly larger /
// smaller (heapq.cuh:17-21, 53-57).
template <bool kLarger>
__device__ __forceinline__ int warp_walk(const HeapEntry *h, int n, int lane, const WalkLane &L) {
    int a = 1;
    while (2 * a <= n) {
        const int node = (a << L.depth) + L.off;
        const bool valid = lane < 31 && node <= n;
        const bool has_child = valid && 2 * node <= n;
        bool right = false;
        if (has_child) {
            const int4 p = *reinterpret_cast<const int4 *>(h + 2 * node);
            const float lk = __int_as_float(p.x), rk = __int_as_float(p.z);
            right = (2 * node + 1 <= n) && (kLarger ? rk > lk : rk < lk);
        }
        const unsigned B = __ballot_sync(kAll, right);
        const unsigned HC = __ballot_sync(kAll, has_child);
        const unsigned P = __ballot_sync(kAll, valid && (B & L.care) == L.want);
        const int rs = 32 - __clz(P);  // deepest node of the path inside the sub-tree (P has bit 0)
        const int ds = 31 - __clz(rs);
        const int ns = (a << ds) + (rs - (1 << ds));
        a = ((HC >> (rs - 1)) & 1u) ? 2 * ns + static_cast<int>((B >> (rs - 1)) & 1u) : ns;
    }
    return a;
}

// heapq.cuh:13-29: the root sinks while a child is strictly smaller.  `me` takes
// the root's place first (callers have read the root if they need it).
__device__ __forceinline__ void warp_sink(HeapEntry *h, int n, HeapEntry me, int lane,
                                          const WalkLane &L) {
    const int leaf = warp_walk<false>(h, n, lane, L);
    const int D = 31 - __clz(leaf);       // path nodes below the root
    const bool on = lane < D;
    const int node = on ? leaf >> (D - 1 - lane) : 1;   // lane l: the path node at depth l + 1
    const HeapEntry e = h[node];
    const unsigned m = __ballot_sync(kAll, on && e.k < me.k);
    const int cnt = __ffs(~m) - 1;        // children that move up one level
    if (lane < cnt) h[node >> 1] = e;
    if (lane == 0) h[cnt == 0 ? 1 : leaf >> (D - cnt)] = me;
    __syncwarp();
}

// heapq.cuh:38-45
__device__ __forceinline__ HeapEntry warp_pop(HeapEntry *h, int n, int lane, const WalkLane &L) {
    const HeapEntry out = h[1];
    __syncwarp();
    warp_sink(h, n, HeapEntry{CUDART_INF_F, -1}, lane, L);
    return out;
}

// heapq.cuh:79-87
__device__ __forceinline__ void warp_pushpop(HeapEntry *h, int n, float k, int32_t v, int lane,
                                             const WalkLane &L) {
    if (k <= h[1].k) return;
    __syncwarp();
    warp_sink(h, n, HeapEntry{k, v}, lane, L);
}

// heapq.cuh:47-77: the leaf at the end of the larger-child walk is replaced if the
// new key is smaller, then sifted up while the parent is strictly larger.
__device__ __forceinline__ void warp_replace(HeapEntry *h, int n, float k, int32_t v, int lane,
                                             const WalkLane &L) {
    const int leaf = warp_walk<true>(h, n, lane, L);
    if (k >= h[leaf].k) return;
    const int D = 31 - __clz(leaf);
    const bool on = lane < D;
    const HeapEntry e = h[on ? leaf >> (lane + 1) : 1];  // lane l: the ancestor l + 1 levels up
    const unsigned m = __ballot_sync(kAll, on && e.k > k);
    const int cnt = __ffs(~m) - 1;        // ancestors that move down one level
    if (lane < cnt) h[leaf >> lane] = e;
    if (lane == 0) h[leaf >> cnt] = HeapEntry{k, v};
    __syncwarp();
}

// ---- distances: one warp per row, two rows in flight ----------------------------
__device__ __forceinline__ float ref_stripe(float acc, float4 c, float4 p) {
    const float dx = __fsub_rn(c.x, p.x), dy = __fsub_rn(c.y, p.y);
    const float dz = __fsub_rn(c.z, p.z), dw = __fsub_rn(c.w, p.w);
    acc = __fadd_rn(acc, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
    return __fadd_rn(acc, __fmaf_rn(dz, dz, __fmul_rn(dw, dw)));
}

__device__ __forceinline__ float butterfly(float acc) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(kAll, acc, off));
    return acc;
}

// Squared distances of the query to rows r0 and r1 over dims [from, d); every lane
// returns both sums.  Three stripes of each row are loaded before any arithmetic.
__device__ __forceinline__ void two_rows(const float *__restrict__ r0, const float *__restrict__ r1,
                                         const float *q_s, int d, int from, int lane, float &o0,
                                         float &o1) {
    float a0 = 0.0f, a1 = 0.0f;
    for (int o = from + 4 * lane; o < d; o += 384) {
        float4 x0[3], x1[3];
#pragma unroll
        for (int m = 0; m < 3; ++m) {
            const bool in = o + 128 * m < d;
            x0[m] = in ? __ldg(reinterpret_cast<const float4 *>(r0 + o + 128 * m))
                       : make_float4(0, 0, 0, 0);
            x1[m] = in ? __ldg(reinterpret_cast<const float4 *>(r1 + o + 128 * m))
                       : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int m = 0; m < 3; ++m) {
            if (o + 128 * m < d) {
                const float4 qa = *reinterpret_cast<const float4 *>(q_s + o + 128 * m);
                a0 = ref_stripe(a0, qa, x0[m]);
                a1 = ref_stripe(a1, qa, x1[m]);
            }
        }
    }
    o0 = butterfly(a0);
    o1 = butterfly(a1);
}

// One row over dims [from, d) with six stripes (768 floats) loaded before any
// arithmetic: a row of up to 3 KB makes a single round trip.  Same order of
// additions as two_rows.
__device__ __forceinline__ float one_row(const float *__restrict__ r0, const float *q_s, int d,
                                         int from, int lane) {
    float a0 = 0.0f;
    for (int o = from + 4 * lane; o < d; o += 768) {
        float4 x0[6];
#pragma unroll
        for (int m = 0; m < 6; ++m)
            x0[m] = o + 128 * m < d ? __ldg(reinterpret_cast<const float4 *>(r0 + o + 128 * m))
                                    : make_float4(0, 0, 0, 0);
#pragma unroll
        for (int m = 0; m < 6; ++m)
            if (o + 128 * m < d)
                a0 = ref_stripe(a0, *reinterpret_cast<const float4 *>(q_s + o + 128 * m), x0[m]);
    }
    return butterfly(a0);
}

// A third row rides along without registers: cp.async copies it into the warp's
// own staging buffer while the two register rows make their round trips; every
// lane later reads back exactly the 16-byte pieces it copied itself.
__device__ __forceinline__ void row_to_stage(float *stage, const float *__restrict__ row, int d,
                                             int from, int lane) {
    for (int o = from + 4 * lane; o < d; o += 128) {
        const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(stage + o));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(row + o) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__device__ __forceinline__ float staged_row(const float *stage, const float *q_s, int d, int from,
                                            int lane) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    float a = 0.0f;
    for (int o = from + 4 * lane; o < d; o += 128)
        a = ref_stripe(a, *reinterpret_cast<const float4 *>(q_s + o),
                       *reinterpret_cast<const float4 *>(stage + o));
    return butterfly(a);
}

struct RefShared {
    float *q;          // [d]
    HeapEntry *open;   // [2H + 2]
    HeapEntry *buf;    // [H + 2]
    int32_t *c_id;     // [n_cand] seeds of the running stage, then its output
    float *c_d;
    int32_t *nb_id;    // [2][kMaxDegree] unvisited neighbours of an expanded node
    float *nb_d;       //                 (two expansions are in flight)
    float *stage;      // [warps][d] one staged vector row per warp
};

// What the heap warp publishes after a pop, and the gather side's guess.
struct RefCtl {
    unsigned long long m1, m2;  // brief_search: the two smallest seeds, key bits << 32 | index
    int c1, c2;                 //               other seeds with the same distances
    int pop_u[2];       // node popped for expansion i (slot i & 1), -1: the search ends
    float root_k[2];    // open heap's root right after that pop
    int root_v[2];
    int guess[2];       // node the gather warps prepared expansion i for
    int n_new[2];       // unvisited neighbours found for expansion i
    int tie;            // select_sort_output gave up: run upstream's sequence
    unsigned next;      // the query claimed for the CTA's next round
    int sorted;         // the last select_sort_output wrote its output (strictly ascending)
    int n_taken, n_equal;
    int marker;
};

__device__ __forceinline__ void gather_sync() {  // the gather warps only
    asm volatile("bar.sync 1, %0;" ::"r"(static_cast<int>(blockDim.x) - 32) : "memory");
}

// The gather half of one expansion (traverse_cpu.cpp:105-135 without the heap
// updates): the row of u in order up to its first negative id, unvisited ids
// marked and compacted in row order into buffer p, their full-dimension distances.
// Called by all gather warps.
__device__ __forceinline__ void gather_node(const RefineArgs &A, const RefShared &S,
                                            const RefGraph &G, uint8_t *vis, uint8_t marker,
                                            RefCtl *ctl, int u, int p, int gw, int lane, int *prof,
                                            long long &prof_t) {
    (void)prof; (void)prof_t;
    PA_GTICK(0);  // since the last tick: prediction, barriers, waiting for the heap warp
    int32_t *nb_id = S.nb_id + p * kMaxDegree;
    float *nb_d = S.nb_d + p * kMaxDegree;
    const int d = A.d;
    if (gw == 0) {
        const int64_t row = G.row_of != nullptr ? __ldg(G.row_of + u) : u;
        int count = 0;
        bool ended = row < 0;
        for (int c = 0; c < G.degree; c += 32) {
            const int slot = c + lane;
            int v = -1;
            if (!ended && slot < G.degree)
                v = __ldg(G.nbr + row * G.row_stride + static_cast<int64_t>(slot) * G.elem_stride);
            const unsigned end_mask = __ballot_sync(kAll, v < 0 && v != kDupTag);
            PA_GTICK(1);  // adjacency row
            const int first_end = end_mask ? __ffs(end_mask) - 1 : 32;
            const bool live = lane < first_end && v >= 0;
            bool fresh = false;
            if (live) {
                fresh = vis[v] != marker;
                if (fresh) vis[v] = marker;
            }
            const unsigned m = __ballot_sync(kAll, fresh);
            if (fresh) nb_id[count + __popc(m & ((1u << lane) - 1u))] = v;
            count += __popc(m);
            ended = ended || end_mask != 0;
        }
        if (lane == 0) ctl->n_new[p] = count;
    }
    PA_GTICK(5);  // visited bytes
    gather_sync();
    PA_GTICK(2);
    const int n_new = ctl->n_new[p];
    float *stage = S.stage + (gw + 1) * d;
    const int n_gw = static_cast<int>(blockDim.x >> 5) - 1;  // gather warps
    if (d > 384) {
        // two rows per warp and trip, each in one round trip: one through registers,
        // one staged by cp.async
        for (int j = gw; j < n_new; j += 2 * n_gw) {
            const int j1 = j + n_gw;
            if (j1 < n_new) row_to_stage(stage, A.storage + static_cast<int64_t>(nb_id[j1]) * d, d, 0, lane);
            const float r0 = one_row(A.storage + static_cast<int64_t>(nb_id[j]) * d, S.q, d, 0, lane);
            float r1 = 0.0f;
            if (j1 < n_new) r1 = staged_row(stage, S.q, d, 0, lane);
            if (lane == 0) {
                nb_d[j] = r0;
                if (j1 < n_new) nb_d[j1] = r1;
            }
        }
        PA_GTICK(3);  // vector rows
        return;
    }
    // short rows, three per warp and trip: two through registers, one staged
    for (int j = gw; j < n_new; j += 3 * n_gw) {
        const int j1 = j + n_gw, j2 = j + 2 * n_gw;
        const int v0 = nb_id[j], v1 = j1 < n_new ? nb_id[j1] : v0;
        if (j2 < n_new) row_to_stage(stage, A.storage + static_cast<int64_t>(nb_id[j2]) * d, d, 0, lane);
        float r0, r1;
        two_rows(A.storage + static_cast<int64_t>(v0) * d, A.storage + static_cast<int64_t>(v1) * d,
                 S.q, d, 0, lane, r0, r1);
        float r2 = 0.0f;
        if (j2 < n_new) r2 = staged_row(stage, S.q, d, 0, lane);
        if (lane == 0) {
            nb_d[j] = r0;
            if (j1 < n_new) nb_d[j1] = r1;
            if (j2 < n_new) nb_d[j2] = r2;
        }
    }
}

// The end of traverse_cpu_kernel (traverse_cpu.cpp:139-162) without heap operations.
// Upstream pushes every seed into the result heap (heap_pushpop keeps the H
// smallest distances; one equal to the current worst stays out), pops the H - k_out
// worst entries and stores the others worst first, i.e. ascending.  When the
// distances that matter are pairwise different, that is the n_real smallest of
// (result heap + seeds) in ascending order, whatever the heaps looked like on the
// way.  So: (1) a radix select over the float bit patterns (non-negative floats
// order like their bits; eight 4-bit passes with 16 shared counters) finds the H-th
// smallest distance T, (2) the entries below T and as many of those equal to T as
// still fit are gathered into the open heap's memory (dead by now), (3) a bitonic
// network sorts them, (4) the first n_real are stored.  More entries equal to T than
// fit, two equal distances among the chosen (pads of the result heap, (-1, +inf),
// excepted: they are interchangeable), or a distance that is negative or NaN make
// the outcome depend on upstream's exact sequence: nothing is written then and the
// caller runs that sequence.  Returns true (CTA-uniform) if the output is written.
__device__ __forceinline__ bool select_sort_output(const RefShared &S, int H, int n_seed,
                                                   int n_real, int k_out, RefCtl *ctl) {
    const int tid = threadIdx.x, n_thr = blockDim.x;
    const int N = H + n_seed;
    int *bins = reinterpret_cast<int *>(S.open);  // 16 counters, then the gathered entries
    HeapEntry *a = S.open;
    if (tid == 0) {
        ctl->tie = 0;
        ctl->n_taken = 0;
        ctl->n_equal = 0;
    }
    // (1) the H-th smallest key
    unsigned prefix = 0, mask = 0;
    int want = H, at_T = 0;
    bool bad = false;
    for (int shift = 28; shift >= 0; shift -= 4) {
        __syncthreads();
        if (tid < 16) bins[tid] = 0;
        __syncthreads();
        for (int x = tid; x < N; x += n_thr) {
            float dx;
            if (x < H) {
                dx = -S.buf[1 + x].k;
            } else {
                if (S.c_id[x - H] < 0) continue;
                dx = S.c_d[x - H];
            }
            if (!(dx >= 0.0f)) bad = true;
            const unsigned key = __float_as_uint(dx);
            if ((key & mask) == prefix) atomicAdd(&bins[(key >> shift) & 15u], 1);
        }
        __syncthreads();
        int before = 0, digit = 15;
        bool found = false;
#pragma unroll
        for (int b = 0; b < 16; ++b) {  // every thread, same result
            const int c = bins[b];
            if (!found) {
                if (before + c < want) {
                    before += c;
                } else {
                    digit = b;
                    found = true;
                }
            }
        }
        want -= before;
        at_T = bins[digit];
        prefix |= static_cast<unsigned>(digit) << shift;
        mask |= 15u << shift;
    }
    const unsigned T = prefix;  // `want` of the at_T entries equal to T are needed
    if (at_T > want && T != __float_as_uint(CUDART_INF_F)) bad = true;
    if (bad) ctl->tie = 1;
    __syncthreads();
    if (ctl->tie != 0) return false;
    // (2) gather
    int P = 1;
    while (P < H) P <<= 1;  // P <= 2H - 1 entries fit
    for (int i = H + tid; i < P; i += n_thr) a[i] = HeapEntry{CUDART_INF_F, -1};
    for (int x = tid; x < N; x += n_thr) {
        HeapEntry e;
        if (x < H) {
            e = S.buf[1 + x];
            e.k = -e.k;
        } else {
            e.v = S.c_id[x - H];
            if (e.v < 0) continue;
            e.k = S.c_d[x - H];
        }
        const unsigned key = __float_as_uint(e.k);
        bool take = key < T;
        if (key == T) take = atomicAdd(&ctl->n_equal, 1) < want;
        if (take) a[atomicAdd(&ctl->n_taken, 1)] = e;
    }
    __syncthreads();
    // (3) sort ascending
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < (P >> 1); t += n_thr) {
                const int lo = 2 * t - (t & (stride - 1));  // index with bit `stride` clear
                const int hi = lo + stride;
                const bool up = (lo & size) == 0;
                const HeapEntry x = a[lo], y = a[hi];
                if ((x.k > y.k) == up) {
                    a[lo] = y;
                    a[hi] = x;
                }
            }
            __syncthreads();
        }
    }
    bool tie = false;
    for (int i = tid; i + 1 < H; i += n_thr)
        if (a[i].k == a[i + 1].k && (a[i].v >= 0 || a[i + 1].v >= 0)) tie = true;
    if (tie) ctl->tie = 1;
    __syncthreads();
    if (ctl->tie != 0) return false;
    // (4)
    for (int r = tid; r < n_real; r += n_thr) {
        const HeapEntry e = a[r];
        S.c_id[k_out - n_real + r] = e.v;
        S.c_d[k_out - n_real + r] = e.k;
    }
    return true;
}

// A search of exactly two expansions (the sub-graph stage: REFINE_STEP = 2,
// traverse_cpu.cpp:317-326) without the open heap.  heap_replace only ever drops or
// evicts an entry that is no smaller than the leaf at the end of a larger-child
// walk, and at least four entries of a heap of 32 or more are no larger than that
// leaf (the root, its larger child and that child's sibling, the next node of the
// walk) -- so the two smallest keys ever offered are in the heap when they are
// popped, and with pairwise different keys the two pops are simply: the smallest
// seed, then the smaller of the second-smallest seed and the best neighbour
// admitted during the first expansion.  The result heap is kept exactly as
// upstream keeps it (its worst entry decides admissions and the stop test).
// Whenever the keys that matter are not pairwise different the layout of the open
// heap decides: with equal smallest seeds nothing is done and false is returned (the
// caller runs upstream's sequence); a tie met at the second pop is settled by
// building the open heap after all, in upstream's order, and popping it.
// Called by all threads after the seeds are marked; returns CTA-uniformly.
__device__ __forceinline__ bool brief_search(const RefineArgs &A, const RefShared &S,
                                             const RefGraph &G, uint8_t *vis, uint8_t marker,
                                             int n_seed, RefCtl *ctl, const WalkLane &WL,
                                             int &n_expand, int &n_eval, int *prof,
                                             long long &prof_t) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, n_thr = blockDim.x;
    const int H = A.H;
    constexpr unsigned long long kNone = ~0ull;
    if (tid == 0) {
        ctl->m1 = ctl->m2 = kNone;
        ctl->c1 = ctl->c2 = 0;
        ctl->tie = 0;
    }
    __syncthreads();
    bool bad = false;
    for (int i = tid; i < n_seed; i += n_thr) {
        if (S.c_id[i] < 0) continue;
        const float dist = S.c_d[i];
        if (!(dist >= 0.0f && dist < CUDART_INF_F)) bad = true;
        atomicMin(&ctl->m1, (static_cast<unsigned long long>(__float_as_uint(dist)) << 32) | i);
    }
    if (bad) ctl->tie = 1;
    __syncthreads();
    const unsigned long long m1 = ctl->m1;
    const int i1 = static_cast<int>(m1 & 0xffffffffu);
    for (int i = tid; i < n_seed; i += n_thr) {
        if (S.c_id[i] < 0 || i == i1) continue;
        const unsigned key = __float_as_uint(S.c_d[i]);
        if (key == static_cast<unsigned>(m1 >> 32)) atomicAdd(&ctl->c1, 1);
        atomicMin(&ctl->m2, (static_cast<unsigned long long>(key) << 32) | i);
    }
    __syncthreads();
    if (ctl->tie != 0 || ctl->c1 != 0) return false;  // nothing has been changed
    const unsigned long long m2 = ctl->m2;
    const int i2 = static_cast<int>(m2 & 0xffffffffu);
    for (int i = tid; i < n_seed; i += n_thr) {
        if (S.c_id[i] < 0 || i == i1 || i == i2) continue;
        if (__float_as_uint(S.c_d[i]) == static_cast<unsigned>(m2 >> 32)) atomicAdd(&ctl->c2, 1);
    }
    __syncthreads();
    if (m1 == kNone) return true;  // no seed at all: the first pop ends the search
    // first pop: the smallest seed; the result heap is empty, the stop test passes
    const int u1 = S.c_id[i1];
    if (w > 0) gather_node(A, S, G, vis, marker, ctl, u1, 0, w - 1, lane, prof, prof_t);
    __syncthreads();
    if (w == 0) {
        const int n_new = ctl->n_new[0];
        ++n_expand;
        n_eval += n_new;
        unsigned long long admitted = 0;
        float best = CUDART_INF_F;
        int best_j = -1;
        bool best_twice = false;
        for (int j = 0; j < n_new; ++j) {  // heap_update (:23-39) without the open heap
            const float dist = S.nb_d[j];
            if (dist >= -S.buf[1].k) continue;
            warp_pushpop(S.buf, H, -dist, S.nb_id[j], lane, WL);
            admitted |= 1ull << j;
            if (dist < best) {
                best = dist;
                best_j = j;
                best_twice = false;
            } else if (dist == best) {
                best_twice = true;
            }
        }
        // second pop
        const bool seed_left = m2 != kNone;
        const float seed_k = seed_left ? S.c_d[i2] : CUDART_INF_F;
        int u2 = -1;
        float k2 = CUDART_INF_F;
        bool unsure = false;
        if (best_j >= 0 && (!seed_left || best < seed_k)) {
            u2 = S.nb_id[best_j];
            k2 = best;
            unsure = best_twice;
        } else if (seed_left && (best_j < 0 || seed_k < best)) {
            u2 = S.c_id[i2];
            k2 = seed_k;
            unsure = ctl->c2 != 0;
        } else if (seed_left) {  // equal
            unsure = true;
        }
        if (unsure) {  // upstream's sequence on the open heap
            for (int i = 0; i < n_seed; ++i) {
                const int id = S.c_id[i];
                if (id >= 0) warp_replace(S.open, 2 * H, S.c_d[i], id, lane, WL);
            }
            warp_pop(S.open, 2 * H, lane, WL);
            for (int j = 0; j < n_new; ++j)
                if ((admitted >> j) & 1ull) warp_replace(S.open, 2 * H, S.nb_d[j], S.nb_id[j], lane, WL);
            const HeapEntry nx = warp_pop(S.open, 2 * H, lane, WL);
            u2 = nx.v;
            k2 = nx.k;
        }
        if (u2 >= 0 && k2 >= -S.buf[1].k) u2 = -1;  // :86-90
        if (lane == 0) ctl->pop_u[1] = u2;
    }
    __syncthreads();
    const int u2 = ctl->pop_u[1];
    if (u2 < 0) return true;
    if (w > 0) gather_node(A, S, G, vis, marker, ctl, u2, 1, w - 1, lane, prof, prof_t);
    __syncthreads();
    if (w == 0) {
        const int n_new = ctl->n_new[1];
        const int32_t *nb_id = S.nb_id + kMaxDegree;
        const float *nb_d = S.nb_d + kMaxDegree;
        ++n_expand;
        n_eval += n_new;
        for (int j = 0; j < n_new; ++j) {
            const float dist = nb_d[j];
            if (dist >= -S.buf[1].k) continue;
            warp_pushpop(S.buf, H, -dist, nb_id[j], lane, WL);
        }
    }
    return true;
}

// One call of upstream's traverse_cpu_kernel: seeds in c_id / c_d (n_seed of
// them), the result (k_out entries, ascending behind (-1, -inf) pads) back into
// c_id / c_d.  `from` < d: the seeds' distances are first completed over dims
// [from, d).  Returns expansions and evaluations through n_expand / n_eval
// (warp 0).
__device__ __forceinline__ void search_stage(const RefineArgs &A, const RefShared &S,
                                             const RefGraph &G, uint8_t *vis, uint8_t marker,
                                             int n_seed, int from, int max_iter, int k_out,
                                             bool speculate, bool seeds_sorted, RefCtl *ctl,
                                             int &n_expand, int &n_eval, int *prof,
                                             long long &prof_t) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int d = A.d, H = A.H;
    (void)prof; (void)prof_t;
    // distances completed over the trailing dims (:41-62), in place
    if (from < d) {
        float *stage = S.stage + w * d;
        const int n_w = static_cast<int>(blockDim.x >> 5);
        if (d - from > 384) {  // long rows: one round trip each, two rows per warp and trip
            for (int i = w; i < n_seed; i += 2 * n_w) {
                const int i1 = i + n_w;
                const int id0 = S.c_id[i], id1 = i1 < n_seed ? S.c_id[i1] : -1;
                if (id0 < 0 && id1 < 0) continue;  // warp-uniform
                if (id1 >= 0) row_to_stage(stage, A.storage + static_cast<int64_t>(id1) * d, d, from, lane);
                float r0 = 0.0f, r1 = 0.0f;
                if (id0 >= 0) r0 = one_row(A.storage + static_cast<int64_t>(id0) * d, S.q, d, from, lane);
                if (id1 >= 0) r1 = staged_row(stage, S.q, d, from, lane);
                if (lane == 0) {
                    if (id0 >= 0) S.c_d[i] = __fadd_rn(S.c_d[i], r0);
                    if (id1 >= 0) S.c_d[i1] = __fadd_rn(S.c_d[i1], r1);
                }
            }
        } else {
            for (int i = w; i < n_seed; i += 3 * n_w) {
                const int i1 = i + n_w, i2 = i + 2 * n_w;
                const int id0 = S.c_id[i], id1 = i1 < n_seed ? S.c_id[i1] : -1;
                const int id2 = i2 < n_seed ? S.c_id[i2] : -1;
                if (id0 < 0 && id1 < 0 && id2 < 0) continue;  // warp-uniform
                if (id2 >= 0) row_to_stage(stage, A.storage + static_cast<int64_t>(id2) * d, d, from, lane);
                float r0, r1;
                two_rows(A.storage + static_cast<int64_t>(max(id0, 0)) * d,
                         A.storage + static_cast<int64_t>(max(id1, 0)) * d, S.q, d, from, lane, r0, r1);
                float r2 = 0.0f;
                if (id2 >= 0) r2 = staged_row(stage, S.q, d, from, lane);
                if (lane == 0) {
                    if (id0 >= 0) S.c_d[i] = __fadd_rn(S.c_d[i], r0);
                    if (id1 >= 0) S.c_d[i1] = __fadd_rn(S.c_d[i1], r1);
                    if (id2 >= 0) S.c_d[i2] = __fadd_rn(S.c_d[i2], r2);
                }
            }
        }
    }
    PA_GTICK(4);  // residual distances of the seeds
    // :65-68
    for (int i = tid; i < H + 2; i += blockDim.x) S.buf[i] = HeapEntry{-CUDART_INF_F, -1};
    for (int i = tid; i < 2 * H + 2; i += blockDim.x) S.open[i] = HeapEntry{CUDART_INF_F, -1};
    // :69-79, the marks (their order does not matter; the heap inserts below keep it)
    for (int i = tid; i < n_seed; i += blockDim.x) {
        const int id = S.c_id[i];
        if (id >= 0) vis[id] = marker;
    }
    __syncthreads();
    PA_TICK(0);
    const WalkLane WL = walk_lane(lane);
    const bool brief = max_iter == 2 && !speculate && 2 * H >= 32 && G.degree <= 64 &&
                       brief_search(A, S, G, vis, marker, n_seed, ctl, WL, n_expand, n_eval, prof, prof_t);
    if (!brief && w == 0) {
        if (seeds_sorted && ctl->sorted != 0 && n_seed >= H) {
            // The real seeds are c[n_seed - H ..] in strictly ascending order.  Every
            // key offered to heap_replace is then larger than all keys in the heap:
            // it replaces a +inf leaf and climbs to just below a real entry, or meets
            // a real leaf and is dropped -- which of the two depends on the count of
            // seeds before it only.  Seed 0 ends at heap index 0, seeds 2t - 1 and 2t
            // at the two rightmost nodes of level t (2^(t+1) - 3 and 2^(t+1) - 2,
            // 0-based) while those exist; all later seeds are dropped.  Checked
            // against heap_replace for every heap size and seed count on the host.
            const int t = (lane + 1) >> 1;
            const int pos = lane == 0 ? 0 : (1 << (t + 1)) - 3 + ((lane & 1) ? 0 : 1);
            const int at = n_seed - H + lane;
            if (lane < 25 && pos < 2 * H && at < n_seed && S.c_id[at] >= 0)
                S.open[1 + pos] = HeapEntry{S.c_d[at], S.c_id[at]};
            __syncwarp();
        } else {
            for (int i = 0; i < n_seed; ++i) {
                const int id = S.c_id[i];
                if (id >= 0) warp_replace(S.open, 2 * H, S.c_d[i], id, lane, WL);
            }
        }
    }
    PA_TICK(1);
    // :82-136.  Expansion i uses slot i & 1 of the control block and of the
    // neighbour buffers.  Per expansion one CTA-wide barrier: behind it the heap
    // warp has popped node i (or ended the search) and -- when speculating --
    // the gather warps have prepared the node they expected.
    if (!brief && w == 0) {
        const HeapEntry u = warp_pop(S.open, 2 * H, lane, WL);
        const bool stop = max_iter <= 0 || u.v < 0 || u.k >= -S.buf[1].k;
        if (lane == 0) {
            ctl->pop_u[0] = stop ? -1 : u.v;
            ctl->root_k[0] = S.open[1].k;
            ctl->root_v[0] = S.open[1].v;
            ctl->guess[0] = ctl->guess[1] = -2;
        }
    }
    PA_TICK(2);
    for (int step = 0; step < max_iter && !brief; ++step) {
        const int p = step & 1;
        __syncthreads();
        PA_TICK(4);
        if (step == 0) { PA_GTICK(7); } else { PA_GTICK(6); }  // waiting for the heap warp: seed inserts / a pop
        const int u = ctl->pop_u[p];
        if (u < 0) break;
        if (u != ctl->guess[p]) {  // CTA-uniform: nothing, or something else, was prepared
            if (w > 0) gather_node(A, S, G, vis, marker, ctl, u, p, w - 1, lane, prof, prof_t);
            __syncthreads();
        }
        PA_TICK(3);
        if (w == 0) {
            // heap_update (:23-39) in row order, then the next pop (:84-90)
            const int n_new = ctl->n_new[p];
            const int32_t *nb_id = S.nb_id + p * kMaxDegree;
            const float *nb_d = S.nb_d + p * kMaxDegree;
            ++n_expand;
            n_eval += n_new;
            for (int j = 0; j < n_new; ++j) {
                const float dist = nb_d[j];
                if (dist >= -S.buf[1].k) continue;
                warp_pushpop(S.buf, H, -dist, nb_id[j], lane, WL);
                warp_replace(S.open, 2 * H, dist, nb_id[j], lane, WL);
#if PA_REFINE_PROFILE
                if (PA_REFINE_PROFILE == 1 && threadIdx.x == 0) prof[7] += 1;
#endif
            }
            PA_TICK(5);
            if (step + 1 < max_iter) {
                const HeapEntry nx = warp_pop(S.open, 2 * H, lane, WL);
                const bool stop = nx.v < 0 || nx.k >= -S.buf[1].k;
                if (lane == 0) {
                    ctl->pop_u[p ^ 1] = stop ? -1 : nx.v;
                    ctl->root_k[p ^ 1] = S.open[1].k;
                    ctl->root_v[p ^ 1] = S.open[1].v;
                }
            }
            PA_TICK(2);
        } else if (speculate && step + 1 < max_iter) {
            // the node the next pop returns unless it ends the search: the first
            // new neighbour with the smallest distance if that is below the root
            // the open heap had after this expansion's pop, else that root
            const int n_new = ctl->n_new[p];
            const float *nb_d = S.nb_d + p * kMaxDegree;
            float best = CUDART_INF_F;
            int at = 0x7fffffff;
            for (int j = lane; j < n_new; j += 32) {
                const float dist = nb_d[j];
                if (dist < best) { best = dist; at = j; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ob = __shfl_xor_sync(kAll, best, off);
                const int oa = __shfl_xor_sync(kAll, at, off);
                if (ob < best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            const int guess = best < ctl->root_k[p] ? S.nb_id[p * kMaxDegree + at] : ctl->root_v[p];
            if (tid == 32) ctl->guess[p ^ 1] = guess;
            if (guess >= 0) gather_node(A, S, G, vis, marker, ctl, guess, p ^ 1, w - 1, lane, prof, prof_t);
        }
        PA_TICK(5);
    }
    // :139-162: the seeds join the result heap; all but k_out are dropped; what is
    // left comes out worst first and is stored ascending
    const int n_real = min(k_out, H);
    const bool sorted = select_sort_output(S, H, n_seed, n_real, k_out, ctl);  // CTA-uniform
    if (tid == 0) ctl->sorted = sorted;  // the output is strictly ascending up to its trailing pads
    if (!sorted) {
        if (w == 0) {
            for (int i = 0; i < n_seed; ++i) {
                const int id = S.c_id[i];
                if (id >= 0) warp_pushpop(S.buf, H, -S.c_d[i], id, lane, WL);
            }
            for (int i = k_out; i < H; ++i) warp_pop(S.buf, H, lane, WL);
        }
        __syncthreads();  // the seeds have been read: their slots may be overwritten
        if (w == 0) {
            for (int i = 0; i < n_real; ++i) {
                const HeapEntry e = warp_pop(S.buf, H, lane, WL);
                if (lane == 0) {
                    S.c_id[k_out - i - 1] = e.v;
                    S.c_d[k_out - i - 1] = -e.k;
                }
            }
        }
    }
    // pops of an exhausted heap give (-1, key +inf): the leading pads
    for (int i = tid; i < k_out - n_real; i += blockDim.x) {
        S.c_id[i] = -1;
        S.c_d[i] = -CUDART_INF_F;
    }
    __syncthreads();
    PA_TICK(6);
    PA_GTICK(8);  // merge and output
}

__global__ void __launch_bounds__(kRefThreads, PA_REFINE_MIN_CTAS) refine_kernel(RefineArgs A) {
    extern __shared__ __align__(16) unsigned char ref_smem[];
    __shared__ RefCtl ctl_s;
    RefCtl *ctl = &ctl_s;
    RefShared S;
    S.q = reinterpret_cast<float *>(ref_smem);
    S.open = reinterpret_cast<HeapEntry *>(S.q + A.d);
    S.buf = S.open + 2 * A.H + 2;
    S.c_id = reinterpret_cast<int32_t *>(S.buf + A.H + 2);
    S.c_d = reinterpret_cast<float *>(S.c_id + A.n_cand);
    S.nb_id = reinterpret_cast<int32_t *>(S.c_d + A.n_cand);
    S.nb_d = reinterpret_cast<float *>(S.nb_id + 2 * kMaxDegree);
    S.stage = S.nb_d + 2 * kMaxDegree;
    const int tid = threadIdx.x;
    const int slot = A.slot_begin + blockIdx.x;
    uint8_t *vis = A.marks + static_cast<int64_t>(slot) * A.slot_stride;

    // CTA i starts on query i; whoever finishes claims the next unclaimed query (queries
    // differ several-fold in length, and a launch is over when its last CTA is)
    for (int64_t b = blockIdx.x; b < A.batch;) {
        // next marker of this slot; the array is wiped when the markers run out
        // (bitmask.hpp:17-36 does the same on wrap-around)
        if (tid == 0) ctl->marker = A.epoch[slot] + 1;
        __syncthreads();
        int marker = ctl->marker;
        if (marker > 254) {
            uint4 *p = reinterpret_cast<uint4 *>(vis);
            for (int64_t i = tid; i < A.slot_stride / 16; i += blockDim.x)
                p[i] = make_uint4(0, 0, 0, 0);
            marker = 1;
        }
        __syncthreads();
        if (tid == 0) A.epoch[slot] = marker;

        for (int i = tid; i < A.d; i += blockDim.x) S.q[i] = A.query[b * A.ldq + i];
        for (int i = tid; i < A.n_cand; i += blockDim.x) {
            const int64_t id = A.cand_I[b * A.n_cand + i];
            S.c_id[i] = (id < 0 || id >= A.n_nodes) ? -1 : static_cast<int32_t>(id);
            S.c_d[i] = A.cand_D[b * A.n_cand + i];
        }
        __syncthreads();
        int st[4] = {0, 0, 0, 0};
        int prof[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
        long long prof_t = 0;
#if PA_REFINE_PROFILE
        prof_t = pinned_clock();
#endif
        // stage 2 (traverse_cpu.cpp:317-326): sub-graph, REFINE_STEP expansions
        search_stage(A, S, A.sub, vis, static_cast<uint8_t>(marker), A.n_cand, A.d_p,
                     min(2, 2 * A.ef), A.n_cand, false, false, ctl, st[0], st[1], prof, prof_t);
        int k_out = A.n_cand;
        if (A.stages >= 3) {  // stage 3 (:327-336): full graph, same marker
            search_stage(A, S, A.full, vis, static_cast<uint8_t>(marker), A.n_cand, A.d,
                         min(1024, 2 * A.ef), A.k, true, true, ctl, st[2], st[3], prof, prof_t);
            k_out = A.k;
        }
        for (int i = tid; i < k_out; i += blockDim.x) {
            A.out_I[b * k_out + i] = S.c_id[i];
            A.out_D[b * k_out + i] = S.c_d[i];
        }
#if PA_REFINE_PROFILE
        if (A.stats != nullptr && tid == 32)
            for (int i = 0; i < 12; ++i) A.stats[b * 24 + 12 + i] = prof[i];
#endif
        if (A.stats != nullptr && tid == 0) {
#if PA_REFINE_PROFILE
            for (int i = 0; i < 4; ++i) A.stats[b * 24 + i] = st[i];
            for (int i = 0; i < 8; ++i) A.stats[b * 24 + 4 + i] = prof[i];
#else
#pragma unroll
            for (int i = 0; i < 4; ++i) A.stats[b * 4 + i] = st[i];
#endif
        }
        if (tid == 0) ctl->next = atomicAdd(A.claim, 1u);
        __syncthreads();
        b = static_cast<int64_t>(gridDim.x) + ctl->next;
    }
}

// traverse_cpu.cpp:228-254
static int cpu_heap_size_for(int ef) {
    static const int sizes[] = {16, 32, 48, 64, 96, 128, 192, 256, 384, 512, 1024, 2048};
    for (int s : sizes)
        if (ef <= s) return s;
    return -1;
}

// Refinement CTAs one SM holds at ef_search 128 (registers and shared memory): the
// number of visited slots worth having per SM.
int refine_ctas_per_sm(int d_model) {
    const int by_registers = (64 * 1024) / (56 * ref_threads_for(d_model));
    return by_registers < 12 ? by_registers : 12;  // shared memory: about 17 KB per CTA
}

static size_t refine_smem_bytes(int d, int H, int n_cand) {
    // one staged row per warp: a narrow CTA may be launched with up to four warps
    const int warps = max(ref_threads_for(d), 128) / 32;
    return sizeof(float) * d * (1 + warps) + sizeof(HeapEntry) * (3 * H + 4) +
           8 * static_cast<size_t>(n_cand) + 16 * kMaxDegree;
}

static int refine_launch(const RefineArgs &A, int n_slots, cudaStream_t stream) {
    if (A.batch == 0) return PA_OK;
    const size_t smem = refine_smem_bytes(A.d, A.H, A.n_cand);
    static size_t configured[64] = {};
    int dev = 0;
    PA_CUDA_TRY(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && configured[dev] < smem) {
        PA_CUDA_TRY(cudaFuncSetAttribute(refine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
        configured[dev] = smem;
    }
    const unsigned grid = static_cast<unsigned>(min(static_cast<int64_t>(A.batch),
                                                    static_cast<int64_t>(n_slots)));
    int threads = ref_threads_for(A.d);
    if (threads == kRefThreadsNarrow && kRefThreadsNarrow == 96) {
        static int sms[64] = {};
        if (dev >= 0 && dev < 64) {
            if (sms[dev] == 0)
                PA_CUDA_TRY(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
            if (grid <= 9u * static_cast<unsigned>(sms[dev])) threads = 128;
        }
    }
    refine_kernel<<<grid, threads, smem, stream>>>(A);
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

static int refine_check(const void *out_I, const void *out_D, const void *cand_I, const void *cand_D,
                 const float *query, int64_t ldq, const float *storage, const int32_t *packed_nbr,
                 const int32_t *row_of, int n_neighbors, const int32_t *full_nbr, int full_degree,
                 int64_t batch, int64_t n_nodes, int d, int d_p, int n_cand, int ef, int k,
                 int stages) {
    PA_REQUIRE(batch >= 0 && batch <= 0x7fffffff, "batch out of range");
    PA_REQUIRE(stages == 2 || stages == 3, "stages must be 2 (sub-graph stage) or 3 (both)");
    PA_REQUIRE(ef > 0 && cpu_heap_size_for(ef) > 0, "ef_search must be in (0, 2048]");
    PA_REQUIRE(d > 0 && d % 4 == 0 && d_p > 0 && d_p % 4 == 0 && d_p <= d,
               "d_model / d_principle must be multiples of 4 with d_principle <= d_model");
    PA_REQUIRE(ldq >= d && ldq % 4 == 0, "query row stride must be a multiple of 4");
    PA_REQUIRE(n_cand > 0 && n_cand % 4 == 0, "the candidate row must be a positive multiple of 4");
    PA_REQUIRE(n_nodes > 0 && n_nodes < 0x7fffffff, "node ids must fit int32");
    PA_REQUIRE(n_neighbors > 0 && n_neighbors <= kMaxDegree, "n_neighbors must be in (0, 64]");
    if (stages >= 3) {
        PA_REQUIRE(k > 0 && k <= n_cand, "k must be in (0, candidates per query]");
        PA_REQUIRE(full_degree > 0 && full_degree <= kMaxDegree, "full-graph degree must be in (0, 64]");
    }
    PA_REQUIRE(refine_smem_bytes(d, cpu_heap_size_for(ef), n_cand) <= 200 * 1024,
               "d_model, ef_search and the candidate row together exceed the shared memory of a CTA");
    if (batch == 0) return PA_OK;
    PA_REQUIRE(out_I && out_D && cand_I && cand_D && query && storage && packed_nbr && row_of,
               "null pointer");
    PA_REQUIRE(stages < 3 || full_nbr != nullptr, "stage 3 needs the packed full graph");
    PA_REQUIRE(aligned16(query) && aligned16(storage), "query / storage must be 16-byte aligned");
    return PA_OK;
}

static RefineArgs refine_args(int64_t *out_I, float *out_D, const int64_t *cand_I, const float *cand_D,
                       const float *query, int64_t ldq, const float *storage,
                       const int32_t *packed_nbr, const int32_t *row_of, int n_neighbors,
                       const int32_t *full_nbr, int full_degree, int64_t batch, int64_t n_nodes,
                       int d, int d_p, int n_cand, int ef, int k, int stages, uint8_t *marks,
                       int32_t *epoch, int64_t slot_stride, int slot_begin, int32_t *stats) {
    RefineArgs A;
    A.cand_I = cand_I; A.cand_D = cand_D; A.query = query; A.ldq = ldq; A.storage = storage;
    A.n_nodes = n_nodes; A.d = d; A.d_p = d_p;
    A.sub = RefGraph{packed_nbr, row_of, 4 * static_cast<int64_t>(n_neighbors), 4, n_neighbors};
    A.full = RefGraph{full_nbr, nullptr, full_degree, 1, full_degree};
    A.n_cand = n_cand; A.ef = ef; A.H = cpu_heap_size_for(ef); A.k = k; A.stages = stages;
    A.batch = static_cast<int>(batch);
    A.out_I = out_I; A.out_D = out_D; A.marks = marks; A.epoch = epoch;
    A.slot_stride = slot_stride; A.slot_begin = slot_begin; A.stats = stats;
    return A;
}

// ---- full graph, packed: int32 [n_nodes, degree], -1 padded ----------------------
// One thread per node.  A row stops at its first negative id (as the search
// does); an id that repeats an earlier id of the row is dropped (the search would
// find it visited), so rows hold distinct ids.
__global__ void pack_full_kernel(int32_t *__restrict__ out, const int64_t *__restrict__ indptr,
                                 const int64_t *__restrict__ indices, int64_t n_nodes, int degree,
                                 int *__restrict__ error) {
    const int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (u >= n_nodes) return;
    const int64_t lo = indptr[u], hi = indptr[u + 1];
    int32_t *row = out + u * degree;
    int n = 0;
    for (int64_t i = lo; i < hi; ++i) {
        const int64_t v = indices[i];
        if (v < 0) break;
        if (v >= n_nodes) { atomicMax(error, 2); break; }
        bool dup = false;
        for (int j = 0; j < n; ++j) dup = dup || row[j] == static_cast<int32_t>(v);
        if (dup) continue;
        if (n == degree) { atomicMax(error, 1); break; }
        row[n++] = static_cast<int32_t>(v);
    }
    for (; n < degree; ++n) row[n] = -1;
}

}  // namespace pa

extern "C" int pa_cpu_heap_size_for(int ef_search) { return pa::cpu_heap_size_for(ef_search); }

extern "C" int pa_refine_ctas_per_sm(int d_model) { return pa::refine_ctas_per_sm(d_model); }

namespace pa {

// Checks, then one launch on `stream` whose CTAs own pool slots
// [slot_begin, slot_begin + slot_count).
int refine_enqueue(int64_t *out_I, float *out_D, const int64_t *cand_I, const float *cand_D,
                   const float *query, int64_t ldq, const float *storage_full,
                   const int32_t *packed_nbr, const int32_t *row_of, int n_neighbors,
                   const int32_t *full_nbr, int full_degree, int64_t batch, int64_t n_nodes,
                   int d_model, int d_principle, int n_cand, int ef_search, int k, int stages,
                   const pa_visited_pool *pool, int slot_begin, int slot_count, int32_t *stats,
                   cudaStream_t stream) {
    int rc = refine_check(out_I, out_D, cand_I, cand_D, query, ldq, storage_full, packed_nbr,
                          row_of, n_neighbors, full_nbr, full_degree, batch, n_nodes, d_model,
                          d_principle, n_cand, ef_search, k, stages);
    if (rc != PA_OK || batch == 0) return rc;
    if (pool == nullptr) return fail(PA_ERR_STATE, "visited pool is null");
    uint8_t *marks; int32_t *epoch; int64_t slot_stride, pool_nodes; int n_slots;
    pool_view(pool, &marks, &epoch, &slot_stride, &n_slots, &pool_nodes);
    PA_REQUIRE(pool_nodes >= n_nodes, "the visited pool was created for fewer nodes");
    PA_REQUIRE(slot_begin >= 0 && slot_count > 0 && slot_begin + slot_count <= n_slots,
               "slot range outside the visited pool");
    RefineArgs A = refine_args(out_I, out_D, cand_I, cand_D, query, ldq, storage_full, packed_nbr,
                               row_of, n_neighbors, full_nbr, full_degree, batch, n_nodes, d_model,
                               d_principle, n_cand, ef_search, k, stages, marks, epoch, slot_stride,
                               slot_begin, stats);
    A.claim = reinterpret_cast<unsigned *>(epoch + n_slots + slot_begin);
    PA_CUDA_TRY(cudaMemsetAsync(A.claim, 0, sizeof(unsigned), stream));
    return refine_launch(A, slot_count, stream);
}

}  // namespace pa

extern "C" int pa_refine(int64_t *out_I, float *out_D, const int64_t *cand_I, const float *cand_D,
                         const float *query, const float *storage_full, const int32_t *packed_nbr,
                         const int32_t *row_of, int n_neighbors, const int32_t *full_nbr,
                         int full_degree, int64_t batch, int64_t n_nodes, int d_model,
                         int d_principle, int n_cand, int ef_search, int k, int stages,
                         pa_visited_pool *pool, int32_t *stats, void *stream) {
    return pa::refine_enqueue(out_I, out_D, cand_I, cand_D, query, d_model, storage_full,
                              packed_nbr, row_of, n_neighbors, full_nbr, full_degree, batch,
                              n_nodes, d_model, d_principle, n_cand, ef_search, k, stages, pool, 0,
                              pa_visited_pool_slots(pool), stats, static_cast<cudaStream_t>(stream));
}

extern "C" int pa_pack_fullgraph(int32_t *full_nbr, const int64_t *indptr, const int64_t *indices,
                                 int64_t n_nodes, int degree, void *stream_) {
    using namespace pa;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    PA_REQUIRE(n_nodes >= 0 && n_nodes < 0x7fffffff, "node ids must fit int32");
    PA_REQUIRE(degree > 0 && degree <= kMaxDegree, "degree must be in (0, 64]");
    if (n_nodes == 0) return PA_OK;
    PA_REQUIRE(full_nbr && indptr && indices, "null pointer");
    struct ErrorWord {
        int *p = nullptr;
        cudaStream_t s;
        ~ErrorWord() { if (p != nullptr) cudaFreeAsync(p, s); }
    } word;
    word.s = stream;
    PA_CUDA_TRY(cudaMallocAsync(&word.p, sizeof(int), stream));
    PA_CUDA_TRY(cudaMemsetAsync(word.p, 0, sizeof(int), stream));
    pack_full_kernel<<<static_cast<unsigned>((n_nodes + 127) / 128), 128, 0, stream>>>(
        full_nbr, indptr, indices, n_nodes, degree, word.p);
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    int host_error = 0;
    PA_CUDA_TRY(cudaMemcpyAsync(&host_error, word.p, sizeof(int), cudaMemcpyDeviceToHost, stream));
    PA_CUDA_TRY(cudaStreamSynchronize(stream));
    if (host_error == 1)
        return fail(PA_ERR_UNPACKABLE, "a row holds more than `degree` distinct neighbours");
    if (host_error == 2) return fail(PA_ERR_UNPACKABLE, "a neighbour id is out of range");
    return PA_OK;
}

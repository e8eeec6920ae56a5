// Multi-beam graph traversal in the reduced space -- the HBM-gather-bound hot
// loop of the search stage.  One CTA of four warps per query.  The search
// semantics (four beams, heap layouts, bloom hashing, dealing of candidates to
// beams, stop rules, output order) are those of upstream
// extension/traverse_cuda.cu:45-246, executed in ONE fixed interleaving so that
// the result is a deterministic function of the inputs:
//   * the bloom filter is cleared, then seeded with the admitted entries, then
//     used;
//   * in a round the neighbour slots are tested-and-set beam 0 -> 3, 32 slots
//     at a time; a chunk of 32 runs the four hash steps in lock step and within
//     a step lanes hitting the same bit are served in ascending lane order
//     (__match_any_sync elects the first lane, the others see the bit as set);
//   * each heap sees its operations in upstream's order.
//
// Work split inside the CTA:
//   warp 0  "open" warp: pops the four open heaps, commits the bloom probes in
//           slot order, compacts the survivors, and later applies heap_replace
//           to the four open heaps;
//   warp 1  "result" warp: applies heap_pushpop to the four result heaps and
//           writes the output;
//   warp b  (every warp) loads the neighbour row of beam b together with its
//           bloom probes (CSR layout: computes hashes and same-bit elections),
//           so the four rows proceed in parallel;
//   all warps: 16 teams of 8 lanes evaluate the distances of the first 32
//           survivors of a round; the open warp then starts inserting those
//           while the other three warps evaluate the rest.
// A heap operation is executed by a group of 8 lanes, one lane per level of the
// root-to-leaf path, the four beams side by side in one warp.  The path is not
// found by walking keys in shared memory: each heap keeps, in registers, one bit
// per internal node for "right child smaller" and (open heaps) one for "right
// child larger"; following them is a few integer instructions, after which every
// lane derives its own node of the path by a shift (1-based heap indices).  The
// bits of the nodes whose children changed are refreshed with an 8-lane OR per
// word.  The element layout of the heaps is exactly upstream's after every
// operation (heapq.cuh:13-87), which is what makes evictions -- and therefore
// results -- identical.
//
// Two index layouts are served by the same kernel body:
//   CsrLayout    -- upstream's tensors as they are (int64 indptr / indices /
//                   mapping): four dependent loads per hop, kept for drop-in use;
//   PackedLayout -- 16 bytes per neighbour slot, indexed by storage row: int32
//                   global id and storage row (the row is carried through the
//                   open heap) plus the slot's bloom probes -- hash positions and
//                   same-bit elections are properties of the row, so they are
//                   computed when the index is packed: two dependent loads per
//                   hop (neighbour row, vector rows) and no hashing in the loop.
#include "pa_common.cuh"

namespace pa {

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
    const int4 *nbr;        // [n_storage, n_nb] {global id, storage row, bloom probe (2 words)}
    const int32_t *row_of;  // [n_nodes]
    const float *storage;
    int64_t n_nodes;
};

constexpr int kThreads = kBeams * 32;
// CTAs per SM the kernel is compiled for (register cap 65536 / (128 * n)): 7 is
// right when a batch is one wave (1024 queries on 148 SMs = 6.9 CTAs per SM).
#ifndef PA_MIN_CTAS
#define PA_MIN_CTAS 7
#endif
constexpr int kGroup = 8;  // lanes per heap operation
template <int H> constexpr int kHeapRow = H + kGroup;  // heap + the group's spare slots
constexpr unsigned kFull = 0xffffffffu;

template <int H> struct HeapShape {
    static constexpr int kLog = (H == 32) ? 5 : (H == 64) ? 6 : (H == 128) ? 7 : 8;
    // words covering the bits of nodes 1 .. H/2-1 (node H/2 has one child: bit 0)
    static constexpr int kWords = H <= 64 ? 1 : H / 64;
};

// ---- comparison-bit words --------------------------------------------------
// Bit n of a set belongs to heap node n (1-based); only nodes 1 .. H/2-1 (two
// children) ever carry a set bit.  Nodes of levels 0-4 live in word 0, level 5
// in word 1, level 6 in words 2 and 3.

template <int I, int W>
__device__ __forceinline__ uint32_t word_of(const uint32_t (&w)[W]) {
    if constexpr (I < W) return w[I];
    else return 0u;
}

// bit of node n, n < 32 * W
template <int W>
__device__ __forceinline__ uint32_t bit_at(const uint32_t (&w)[W], unsigned n) {
    uint32_t word = w[0];
    if constexpr (W == 2) word = (n & 32u) ? w[1] : w[0];
    if constexpr (W == 4) {
        const uint32_t lo = (n & 32u) ? w[1] : w[0], hi = (n & 32u) ? w[3] : w[2];
        word = (n & 64u) ? hi : lo;
    }
    return (word >> (n & 31u)) & 1u;
}

// Leaf reached from the root by following the bits.
template <int H, int W>
__device__ __forceinline__ unsigned follow_bits(const uint32_t (&w)[W]) {
    // two dependent instructions per level: a funnel shift (it takes the shift
    // count modulo 32 by itself) and one logic op merging the bit into 2n
    unsigned n = 1;
#pragma unroll
    for (int l = 0; l < HeapShape<H>::kLog - 1; ++l) {
        uint32_t word;
        if (l < 5) word = w[0];
        else if (l == 5) word = word_of<1, W>(w);
        else word = (n & 32u) ? word_of<3, W>(w) : word_of<2, W>(w);
        n = (n << 1) | (__funnelshift_r(word, 0u, n) & 1u);
    }
    return n == H / 2 ? static_cast<unsigned>(H) : n;  // node H/2 has one child only
}

// OR over the 8 lanes of a group.  Warp collectives are always issued with the
// full-warp mask here: on sm_100 the sub-warp forms (a vote, shuffle or redux
// whose member mask names 8 lanes) cost several hundred cycles each, the
// full-mask forms a few tens; the groups are carved out of the full-warp result
// (shift + mask for votes, width-8 shuffles, an xor butterfly for the OR).
__device__ __forceinline__ uint32_t group_or(uint32_t mine) {
    mine |= __shfl_xor_sync(kFull, mine, 1);
    mine |= __shfl_xor_sync(kFull, mine, 2);
    mine |= __shfl_xor_sync(kFull, mine, 4);
    return mine;
}

// XOR `mine` (a single bit, or 0) into the word that holds node n, combined
// over the 8 lanes of a group.
template <int W>
__device__ __forceinline__ void flip_bits(uint32_t (&w)[W], uint32_t mine, unsigned n) {
    if constexpr (W == 1) {
        w[0] ^= group_or(mine);
    } else {
#pragma unroll
        for (int i = 0; i < W; ++i)
            w[i] ^= group_or((n >> 5) == static_cast<unsigned>(i) ? mine : 0u);
    }
}

struct GroupCtx {
    unsigned g;      // lane within the group = level handled
    unsigned gshift; // first lane of this group
};

// ---- heap operations, one group of 8 lanes per heap --------------------------
// K / V: the heap's arrays in shared memory (0-based storage of 1-based nodes),
// followed by one spare slot per lane of the group (kHeapRow entries in all).
// sb / lb: "right child smaller" / "right child larger" bits.

// Puts (k, v) at the root and sinks it (upstream __heapify_up, heapq.cuh:13-29).
// Used for heap_pushpop (after its root test) and heap_pop (k = +inf).
// The operation comes in two halves so that a caller running many of them can
// issue the loads of the next path while it still decides which key to insert:
// sink_load reads what lies along the path the bits point to (it depends on the
// heap only), sink_apply moves the keys and refreshes the bits.  sink_apply
// returns the new root key (group-uniform; meaningful only for active groups).
template <typename V> struct SinkPath {
    unsigned node;  // this lane's node on the path (level g + 1), 2 if none
    bool in;        // the path reaches this lane's level
    float a, sk;    // key of the node, key of its sibling
    V av;
};

template <int H, int W, typename V>
__device__ __forceinline__ SinkPath<V> sink_load(const float *K, const V *Vv,
                                                 const uint32_t (&sb)[W], const GroupCtx &c) {
    SinkPath<V> p;
    const unsigned leaf = follow_bits<H, W>(sb);
    const unsigned L = 31u - __clz(leaf);
    const unsigned t = c.g + 1u;  // this lane's level on the path
    p.in = t <= L;
    p.node = p.in ? (leaf >> (L - t)) : 2u;
    const bool has_sib = p.node < static_cast<unsigned>(H);  // node H has no sibling
    p.a = K[p.node - 1];
    p.av = Vv[p.node - 1];
    p.sk = K[(has_sib ? (p.node ^ 1u) : p.node) - 1];
    return p;
}

template <int H, int W, bool kHasLb, typename V>
__device__ __forceinline__ float sink_apply(float *K, V *Vv, uint32_t (&sb)[W], uint32_t (&lb)[W],
                                            const GroupCtx &c, const SinkPath<V> &p, bool active,
                                            float k, V v) {
    const unsigned t = c.g + 1u;  // this lane's level on the path
    const unsigned node = p.node;
    const bool on = active && p.in;
    const bool sib_ok = on && node < static_cast<unsigned>(H);
    const float a = on ? p.a : CUDART_INF_F;
    // children strictly smaller than the moving key move up one level
    const unsigned cm = (__ballot_sync(kFull, on && a < k) >> c.gshift) & 0xffu;
    const unsigned cnt = __ffs(~cm) - 1;  // number of leading levels that move
    const float a_next = __shfl_down_sync(kFull, a, 1, kGroup);
    const float a_first = __shfl_sync(kFull, a, 0, kGroup);
    const bool moves = on && t <= cnt;
    // Stores are unconditional: a lane with nothing to write aims at its own
    // spare slot behind the heap.  A store under a lane-dependent condition
    // makes the warp diverge, which costs far more than the store.
    const unsigned spare = static_cast<unsigned>(H) + c.g;
    const unsigned up = moves ? (node >> 1) - 1 : spare;
    K[up] = a; Vv[up] = p.av;
    // cnt == 0: the new element stays at the root (written by level-1 lane)
    const unsigned at = (active && t == max(cnt, 1u)) ? (cnt == 0 ? 1u : node) - 1 : spare;
    K[at] = k; Vv[at] = v;
    // refresh the bits of the parents of the moved nodes (path levels 0 .. cnt-1)
    const float nk = (t == cnt) ? k : a_next;  // new key at this lane's node
    const bool odd = node & 1u;
    const float left = odd ? p.sk : nk, right = odd ? nk : p.sk;
    const unsigned parent = node >> 1;
    const bool upd = moves && sib_ok;
    const uint32_t s_flip = (right < left) != (bit_at<W>(sb, parent) != 0);
    flip_bits<W>(sb, (upd && s_flip) ? (1u << (parent & 31u)) : 0u, parent);
    if constexpr (kHasLb) {
        const uint32_t l_flip = (right > left) != (bit_at<W>(lb, parent) != 0);
        flip_bits<W>(lb, (upd && l_flip) ? (1u << (parent & 31u)) : 0u, parent);
    }
    __syncwarp();
    return cnt == 0 ? k : a_first;
}

template <int H, int W, bool kHasLb, typename V>
__device__ __forceinline__ float group_sink(float *K, V *Vv, uint32_t (&sb)[W], uint32_t (&lb)[W],
                                            const GroupCtx &c, bool active, float k, V v) {
    const SinkPath<V> p = sink_load<H, W, V>(K, Vv, sb, c);
    return sink_apply<H, W, kHasLb, V>(K, Vv, sb, lb, c, p, active, k, v);
}

// upstream heap_replace (heapq.cuh:47-77): walk to a leaf along the larger
// child, give up if the new key is not smaller than that leaf, else overwrite it
// and sift up while the parent is strictly larger.  replace_load reads the
// ancestors of `leaf` (the leaf the walk ends in) and the key of that leaf, the
// acceptance limit; replace_apply is the second half, `accept` saying whether
// this group's key passed the test against the limit.
template <typename V> struct ReplacePath {
    unsigned L, child;  // level of the leaf; this lane's path child (level g + 1), 2 if none
    bool in;            // the path has an ancestor at this lane's level
    float b, sk, limit; // ancestor key, key of the path child's sibling, key of the leaf
    V bv;
};

template <int H, typename V>
__device__ __forceinline__ ReplacePath<V> replace_load(const float *K, const V *Vv,
                                                       const GroupCtx &c, unsigned leaf) {
    ReplacePath<V> p;
    p.L = 31u - __clz(leaf);
    p.in = c.g < p.L;  // ancestors: levels 0 .. L-1
    p.child = p.in ? (leaf >> (p.L - c.g - 1u)) : 2u;
    const bool has_sib = p.child < static_cast<unsigned>(H);
    p.b = K[(p.child >> 1) - 1];
    p.bv = Vv[(p.child >> 1) - 1];
    p.sk = K[(has_sib ? (p.child ^ 1u) : p.child) - 1];
    p.limit = K[leaf - 1];
    return p;
}

template <int H, int W, typename V>
__device__ __forceinline__ void replace_apply(float *K, V *Vv, uint32_t (&sb)[W],
                                              uint32_t (&lb)[W], const GroupCtx &c, unsigned leaf,
                                              const ReplacePath<V> &p, bool accept, float k, V v) {
    const unsigned L = p.L;
    const unsigned t = c.g;  // ancestors: levels 0 .. L-1
    const bool on = accept && p.in;
    const unsigned child = p.child;
    const unsigned node = child >> 1;
    const bool has_sib = child < static_cast<unsigned>(H);
    const float b = p.b;
    // ancestors strictly larger than the new key move down one level
    const unsigned cm = (__ballot_sync(kFull, on && b > k) >> c.gshift) & 0xffu;
    const unsigned s = cm ? (__ffs(cm) - 1) : L;  // level where the new element lands
    const bool moves = on && t >= s;
    // unconditional stores, spare slot for lanes with nothing to write (see sink_apply)
    const unsigned spare = static_cast<unsigned>(H) + c.g;
    const unsigned down = moves ? child - 1 : spare;
    K[down] = b; Vv[down] = p.bv;
    // s == L: nothing moves, the new element replaces the leaf (level L-1 lane)
    const unsigned at = (accept && t == min(s, L - 1u)) ? (s == L ? leaf : node) - 1 : spare;
    K[at] = k; Vv[at] = v;
    // parents whose path child changed: levels max(s-1, 0) .. L-1
    const float nk = (t + 1u == s) ? k : b;  // new key of this lane's path child
    const bool odd = child & 1u;
    const float left = odd ? p.sk : nk, right = odd ? nk : p.sk;
    const bool upd = on && t + 1u >= s && has_sib;
    const bool s_flip = (right < left) != (bit_at<W>(sb, node) != 0);
    const bool l_flip = (right > left) != (bit_at<W>(lb, node) != 0);
    flip_bits<W>(sb, (upd && s_flip) ? (1u << (node & 31u)) : 0u, node);
    flip_bits<W>(lb, (upd && l_flip) ? (1u << (node & 31u)) : 0u, node);
    __syncwarp();
}

template <int H, int W, typename V>
__device__ __forceinline__ void group_replace_at(float *K, V *Vv, uint32_t (&sb)[W],
                                                 uint32_t (&lb)[W], const GroupCtx &c,
                                                 unsigned leaf, bool accept, float k, V v) {
    const ReplacePath<V> p = replace_load<H, V>(K, Vv, c, leaf);
    replace_apply<H, W, V>(K, Vv, sb, lb, c, leaf, p, accept, k, v);
}

template <int H, int W, typename V>
__device__ __forceinline__ void group_replace(float *K, V *Vv, uint32_t (&sb)[W],
                                              uint32_t (&lb)[W], const GroupCtx &c, bool active,
                                              float k, V v) {
    const unsigned leaf = follow_bits<H, W>(lb);
    const bool accept = active && k < K[leaf - 1];
    if (!__any_sync(kFull, accept)) return;
    group_replace_at<H, W>(K, Vv, sb, lb, c, leaf, accept, k, v);
}

// ---- distance (upstream traverse_cuda.cu:18-43) -------------------------------
// Eight lanes; lane t owns floats [32m + 4t, 32m + 4t + 4);
// acc += fma(dx,dx,dy*dy); acc += fma(dz,dz,dw*dw); then the shuffle tree 4, 2, 1.
__device__ __forceinline__ float stripe(float acc, float4 c, float4 p) {
    const float dx = __fsub_rn(c.x, p.x), dy = __fsub_rn(c.y, p.y);
    const float dz = __fsub_rn(c.z, p.z), dw = __fsub_rn(c.w, p.w);
    acc = __fadd_rn(acc, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
    return __fadd_rn(acc, __fmaf_rn(dz, dz, __fmul_rn(dw, dw)));
}

__device__ __forceinline__ float team_reduce(float acc) {
#pragma unroll
    for (int off = kTeam / 2; off > 0; off >>= 1)
        acc = __fadd_rn(acc, __shfl_down_sync(kFull, acc, off, kTeam));
    return acc;
}

// ---- bloom -----------------------------------------------------------------------
// One chunk of 32 neighbours, test-and-set in the fixed order, in two parts.
// The probes (bloom_prepare, or read from the packed index): the four bit
// positions of this lane's node and, per hash step, whether this lane is the
// first (lowest) lane of the chunk that touches its bit in that step.
// bloom_commit: the serial part -- per step the elected lanes
// atomically set their bit and learn whether it was set before; a lane that was
// not elected has a lower lane setting the very same bit in the same step, so it
// sees the bit as set.  Returns true for lanes whose node was already present
// (or is not a node).
__device__ __forceinline__ bool bloom_commit(uint32_t *bloom, const BloomProbe &p) {
    bool found = true;
#pragma unroll
    for (int s = 0; s < kFnvSteps; ++s) {
        // a lane that is not elected ORs in nothing and passes: no branch
        const uint32_t bit = ((p.elected >> s) & 1u) << (p.pos[s] & 31);
        const uint32_t old = atomicOr(&bloom[p.pos[s] >> 5], bit);
        found = found && (old & bit) == bit;
        __syncwarp();
    }
    return found;
}

__device__ __forceinline__ void bloom_insert(uint32_t *bloom, int32_t v) {
    uint32_t h = kFnvOffset;
#pragma unroll
    for (int s = 0; s < kFnvSteps; ++s) {
        h = fnv1a_32(static_cast<uint32_t>(v), h);
        const uint32_t p = h & (kBloomBits - 1);
        atomicOr(&bloom[p >> 5], 1u << (p & 31));
    }
}

// What the open warp publishes about a beam's popped node.
struct PopSlot {
    int32_t node, row;
    int64_t lo;
    int len;
    bool fetch;
};

__device__ __forceinline__ void pair_sync() {  // warps 0 and 1 only
    asm volatile("bar.sync 1, 64;" ::: "memory");
}

// Candidates are dealt to the beams four at a time (candidate j -> beam
// (j / 4) mod 4); beam 0 always holds the most.
__device__ __forceinline__ int deal_index(int s, int beam) {
    return 16 * (s >> 2) + 4 * beam + (s & 3);
}
__device__ __forceinline__ int deal_count(int n, int beam) {
    return 4 * (n >> 4) + min(4, max((n & 15) - 4 * beam, 0));
}

// Next candidate of this group's beam, at or after position `s` of the beam's
// list, whose distance is below `limit`; the group examines eight candidates at
// a time.  Returns the position (>= count if there is none).  Between two
// accepted heap operations the acceptance limit of a heap does not change, so
// skipping the candidates that fail it is exactly what running the operation on
// each of them would do.
__device__ __forceinline__ int next_below(const float *cand_d, const GroupCtx &c, int beam,
                                          int s, int count, float limit) {
    bool searching = s < count;
    while (__any_sync(kFull, searching)) {
        const int sc = s + static_cast<int>(c.g);
        const float dist = (searching && sc < count) ? cand_d[deal_index(sc, beam)] : CUDART_INF_F;
        const unsigned m = (__ballot_sync(kFull, dist < limit) >> c.gshift) & 0xffu;
        if (searching) {
            if (m) { s += __ffs(m) - 1; searching = false; }
            else { s += kGroup; searching = s < count; }
        }
    }
    return s;
}

// The same search over a beam's list held in registers (lists of at most 32
// candidates): lane g of the group holds the distances at positions g, g + 8,
// g + 16 and g + 24 (+inf past the end).  Returns the positions whose distance
// is below `limit` as a bit mask.
__device__ __forceinline__ unsigned below_mask(const float (&cd)[4], float limit,
                                               const GroupCtx &c) {
    unsigned m = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k)
        m |= ((__ballot_sync(kFull, cd[k] < limit) >> c.gshift) & 0xffu) << (8 * k);
    return m;
}
// Distance at position p of the list (p group-uniform).
__device__ __forceinline__ float list_at(const float (&cd)[4], unsigned p) {
    float mine = cd[0];
    if ((p >> 3) == 1u) mine = cd[1];
    if ((p >> 3) == 2u) mine = cd[2];
    if ((p >> 3) == 3u) mine = cd[3];
    return __shfl_sync(kFull, mine, p & 7u, kGroup);
}

template <int H, int CH, class Layout>
__global__ void __launch_bounds__(kThreads, PA_MIN_CTAS)
traverse_kernel(Layout L, int64_t *__restrict__ out_I, float *__restrict__ out_D,
                const float *__restrict__ query, const int64_t *__restrict__ init_I,
                const float *__restrict__ init_D, int d, int64_t ldq, int n_init, int ef,
                int32_t *__restrict__ stats) {
    constexpr int W = HeapShape<H>::kWords;
    constexpr int n_nb = 32 * CH;
    __shared__ uint32_t bloom[kBloomWords];
    __shared__ float open_key[kBeams][kHeapRow<H>];
    __shared__ int2 open_val[kBeams][kHeapRow<H>];  // {global id, storage row}
    __shared__ float res_key[kBeams][kHeapRow<H>];
    __shared__ int32_t res_id[kBeams][kHeapRow<H>];
    // survivors {global id, storage row} and their distances; the last 32 entries
    // are spare slots, one per lane, for stores that have nothing to write
    constexpr int kSpare = kBeams * n_nb;
    __shared__ int2 slots[kBeams * n_nb + 32];
    __shared__ float cand_d[kBeams * n_nb + 32];
    __shared__ int n_work_s;
    __shared__ uint2 probe_s[kBeams * n_nb];  // packed bloom probes of a round's slots
    __shared__ PopSlot pop_s[kBeams];
    __shared__ unsigned again_s[2];
    __shared__ int stat_s[4];
    extern __shared__ __align__(16) float q_s[];

    const int lane = threadIdx.x & 31;
    const int w = threadIdx.x >> 5;
    const int64_t b = blockIdx.x;
    GroupCtx gc;
    gc.g = lane & 7;
    const int beam = lane >> 3;  // heap this lane's group works on
    gc.gshift = beam * kGroup;

    for (int i = threadIdx.x; i < kBloomWords; i += kThreads) bloom[i] = 0;
    for (int i = threadIdx.x; i < d; i += kThreads) q_s[i] = query[b * ldq + i];
    for (int i = threadIdx.x; i < kBeams * H; i += kThreads) {
        open_key[i / H][i % H] = CUDART_INF_F;
        open_val[i / H][i % H] = make_int2(-1, -1);
        res_key[i / H][i % H] = -CUDART_INF_F;
        res_id[i / H][i % H] = -1;
    }
    if (threadIdx.x < 4) stat_s[threadIdx.x] = 0;
    if (threadIdx.x < 2) again_s[threadIdx.x] = 0;
    __syncthreads();

    float *okey = open_key[beam];
    int2 *oval = open_val[beam];
    float *rkey = res_key[beam];
    int32_t *rid = res_id[beam];
    uint32_t o_sb[W], o_lb[W], r_sb[W];  // all keys equal at start: all bits 0
#pragma unroll
    for (int i = 0; i < W; ++i) o_sb[i] = o_lb[i] = r_sb[i] = 0;
    float r_root = -CUDART_INF_F;  // warp 1: root key of the result heap
    int n_expand = 0, n_eval = 0, n_rounds = 0;

    // ---- entries (traverse_cuda.cu:96-111): entry i belongs to beam i mod 4 ------
    for (int base = 0; base < n_init; base += kThreads) {
        const int n_here = min(kThreads, n_init - base);
        if (threadIdx.x < n_here) {  // stage ids, rows, distances
            const int i = threadIdx.x;
            const int64_t node = init_I[b * n_init + base + i];
            int32_t row = -1;
            if constexpr (Layout::kPacked) {
                if (node >= 0 && node < L.n_nodes) row = __ldg(L.row_of + node);
            }
            slots[i] = make_int2(node < 0 ? -1 : static_cast<int32_t>(node), row);
            cand_d[i] = init_D[b * n_init + base + i];
        }
        __syncthreads();
        const int steps = (n_here + kBeams - 1) / kBeams;
        if (w == 1) {  // admission test (:99) + result heaps
            for (int s = 0; s < steps; ++s) {
                const int i = s * kBeams + beam;
                const bool have = i < n_here;
                const int2 e = have ? slots[i] : make_int2(-1, -1);
                const float dist = have ? cand_d[i] : 0.0f;
                const bool admit = have && e.x >= 0 && !(dist >= -r_root);
                if (have && !admit && gc.g == 0) slots[i].x = -1;
                const bool push = admit && (-dist > r_root);
                if (__any_sync(kFull, push)) {
                    const float root = group_sink<H, W, false>(rkey, rid, r_sb, r_sb, gc, push,
                                                               -dist, e.x);
                    if (push) r_root = root;
                }
            }
        }
        __syncthreads();
        if (w == 0) {  // open heaps
            for (int s = 0; s < steps; ++s) {
                const int i = s * kBeams + beam;
                const bool have = i < n_here;
                const int2 e = have ? slots[i] : make_int2(-1, -1);
                const float dist = have ? cand_d[i] : 0.0f;
                group_replace<H, W>(okey, oval, o_sb, o_lb, gc, have && e.x >= 0, dist, e);
            }
        } else if (w >= 2) {  // bloom: the union of the admitted entries' bits
            for (int i = 32 * (w - 2) + lane; i < n_here; i += kThreads - 64) {
                const int32_t node = slots[i].x;
                if (node >= 0) bloom_insert(bloom, node);
            }
        }
        __syncthreads();
    }

    // ---- rounds (traverse_cuda.cu:179-226) -----------------------------------------
    for (int step = 0; step < ef; ++step) {
        ++n_rounds;
        // pop until every beam holds a node with an adjacency row, or gives up
        // (:118-134).  Warp 0 pops; each warp then loads the neighbour row of "its"
        // beam and prepares the bloom probes for it, so the four rows, their hashes
        // and their elections proceed in parallel; warp 0 commits them in order.
        int32_t u_node = -1, u_row = -1;   // warp 0: group-uniform per beam
        int64_t u_lo = 0;
        int u_len = 0;
        bool pending = true;
        bool deferred = false;  // warp 0: the popped root of this group's heap is still in place
        for (int outer = 0; outer <= H + 1; ++outer) {  // more than one pass only if a
                                                        // sampled node has an empty row
            if (w == 0) {
                const float bound = -rkey[0];
                bool fetch = false;  // this beam's row must be (re)loaded
                // every pop removes one element, so H + 1 pops always settle a beam;
                // the guard only bounds the loop should that invariant ever be broken
                for (int guard = 0; guard <= H + 1 && __any_sync(kFull, pending); ++guard) {
                    const float top_k = okey[0];
                    const int2 top_v = oval[0];
                    // written as selects: the groups of the warp disagree on all of
                    // these conditions, and a branch on them would split the warp
                    const bool stop = top_v.x < 0 || top_k >= bound;  // the beam gives up
                    bool usable;  // the popped node has an adjacency row
                    int64_t lo = 0, hi = 0;
                    if constexpr (Layout::kPacked) {
                        usable = top_v.y >= 0;
                    } else {
                        // ids come from the caller's entries and graph: one outside
                        // [0, n_nodes) reads row 0's bounds and is treated as a node
                        // without an adjacency row (the packed path drops it at entry)
                        const bool in_range = top_v.x >= 0 && top_v.x < L.n_nodes;
                        const int64_t at = (pending && !stop && in_range) ? top_v.x : 0;
                        lo = __ldg(L.indptr + at);
                        hi = __ldg(L.indptr + min(at + 1, L.n_nodes));  // indptr has n_nodes + 1 entries
                        usable = in_range && lo != hi;
                    }
                    const bool settle = pending && (stop || usable);
                    // The root is known; removing it from the heap (the sink) can wait
                    // when this pop settles every pending beam, which is the usual
                    // case: the popped nodes are published first and the heaps are
                    // repaired while the neighbour rows are on their way.
                    if (__any_sync(kFull, pending && !settle))
                        group_sink<H, W, true>(okey, oval, o_sb, o_lb, gc, pending, CUDART_INF_F,
                                               make_int2(-1, -1));
                    else
                        deferred = pending;
                    u_node = settle ? (stop ? -1 : top_v.x) : u_node;
                    u_row = settle ? (stop ? -1 : top_v.y) : u_row;
                    u_lo = (settle && !stop) ? lo : u_lo;
                    u_len = settle ? (stop ? 0 : static_cast<int>(min(hi - lo, static_cast<int64_t>(n_nb))))
                                   : u_len;
                    fetch = fetch || settle;
                    pending = pending && !settle;
                }
                pending = false;
                // group-uniform values: every lane of the group stores them (same
                // address, same value) rather than one lane under a condition
                pop_s[beam].node = u_node; pop_s[beam].row = u_row;
                pop_s[beam].lo = u_lo; pop_s[beam].len = u_len;
                pop_s[beam].fetch = fetch;
            }
            __syncthreads();
            // The other slot is cleared only now: its last readers (the previous
            // pass, after that pass's second barrier) are all behind the barrier
            // above, and its next writers come after this pass's second barrier.
            if (w == 0) again_s[(outer + 1) & 1] = 0;
            const bool fetch_w = pop_s[w].fetch;  // warp w serves beam w
            const int32_t node_b = pop_s[w].node;
            if constexpr (Layout::kPacked) {
                // ids, rows and ready-made probes in one 16-byte load per lane
                const int32_t row_b = pop_s[w].row;
                int4 e[CH];
#pragma unroll
                for (int c = 0; c < CH; ++c)
                    e[c] = (fetch_w && node_b >= 0)
                        ? __ldg(L.nbr + static_cast<int64_t>(row_b) * n_nb + 32 * c + lane)
                        : make_int4(-1, -1, 0, 0);
                // the open warp repairs its heaps while its row is on its way
                if (w == 0 && __any_sync(kFull, deferred)) {
                    group_sink<H, W, true>(okey, oval, o_sb, o_lb, gc, deferred, CUDART_INF_F,
                                           make_int2(-1, -1));
                    deferred = false;
                }
                if (fetch_w) {
                    // a sampled node whose adjacency row is empty: its beam pops again
                    if (node_b >= 0 && __shfl_sync(kFull, e[0].x, 0) == kEmptyRowTag) {
                        if (lane == 0) atomicOr(&again_s[outer & 1], 1u << w);
                    } else {
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            const int idx = w * n_nb + 32 * c + lane;
                            slots[idx] = make_int2(e[c].x, e[c].y);
                            probe_s[idx] = make_uint2(static_cast<uint32_t>(e[c].z),
                                                      static_cast<uint32_t>(e[c].w));
                        }
                    }
                }
            } else {
                if (w == 0 && __any_sync(kFull, deferred)) {
                    group_sink<H, W, true>(okey, oval, o_sb, o_lb, gc, deferred, CUDART_INF_F,
                                           make_int2(-1, -1));
                    deferred = false;
                }
                if (fetch_w) {
                    const int64_t lo_b = pop_s[w].lo;
                    const int len_b = pop_s[w].len;
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                        const int i = 32 * c + lane;
                        const int32_t v = (node_b >= 0 && i < len_b)
                            ? static_cast<int32_t>(__ldg(L.indices + lo_b + i)) : -1;
                        const int idx = w * n_nb + i;
                        slots[idx] = make_int2(v, -1);
                        probe_s[idx] = probe_pack(bloom_prepare(v, lane));
                    }
                }
            }
            __syncthreads();
            const unsigned again = again_s[outer & 1];
            if (again == 0) break;
            if (w == 0 && ((again >> beam) & 1u)) { pending = true; u_node = -1; }
        }
        if (w == 0) {
            n_expand += __popc(__ballot_sync(kFull, gc.g == 0 && u_node >= 0));
            // bloom test-and-set in slot order, then compaction in place (:137-171):
            // a chunk is read into registers before survivors are written, and
            // survivors always land at or below the chunk's own position
            int off = 0;
            if constexpr (CH == 1) {
                // all loads first, then the 16 atomics back to back, then the
                // compaction: one exposed atomic latency instead of four
                int2 ev[kBeams];
                uint2 pv[kBeams];
#pragma unroll
                for (int bb = 0; bb < kBeams; ++bb) {
                    ev[bb] = slots[bb * n_nb + lane];
                    pv[bb] = probe_s[bb * n_nb + lane];
                }
                uint32_t miss[kBeams];  // nonzero: some probed bit was clear before
#pragma unroll
                for (int bb = 0; bb < kBeams; ++bb) {
                    const BloomProbe pr = probe_unpack(pv[bb]);
                    miss[bb] = 0;
#pragma unroll
                    for (int s = 0; s < kFnvSteps; ++s) {
                        // a lane that is not elected ORs in nothing: no branch
                        const uint32_t bit = ((pr.elected >> s) & 1u) << (pr.pos[s] & 31);
                        miss[bb] |= ~atomicOr(&bloom[pr.pos[s] >> 5], bit) & bit;
                        __syncwarp();
                    }
                }
#pragma unroll
                for (int bb = 0; bb < kBeams; ++bb) {
                    const unsigned m = __ballot_sync(kFull, miss[bb] != 0);
                    slots[miss[bb] != 0 ? off + __popc(m & ((1u << lane) - 1u)) : kSpare + lane] = ev[bb];
                    off += __popc(m);
                }
            } else
#pragma unroll
            for (int bb = 0; bb < kBeams; ++bb) {
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    const int idx = bb * n_nb + 32 * c + lane;
                    const int2 e = slots[idx];
                    const bool seen = bloom_commit(bloom, probe_unpack(probe_s[idx]));
                    const unsigned m = __ballot_sync(kFull, !seen);
                    slots[!seen ? off + __popc(m & ((1u << lane) - 1u)) : kSpare + lane] = e;
                    off += __popc(m);
                }
            }
            n_work_s = off;  // warp-uniform
        }
        __syncthreads();
        const int n_work = n_work_s;
        if (n_work < kTeamsPerWarp) break;  // :182-184, uniform over the CTA

        // distances (:187-204) by teams of 8 lanes, two candidates in flight per
        // team: team `team` of `n_teams` takes candidates j_begin + team,
        // + n_teams, ... below j_end.  The loop bound is the same for every lane of
        // a warp (the team shuffles name the whole warp); lanes past the end carry
        // a false predicate.
        auto distances = [&](int team, int n_teams, int j_begin, int j_end) {
            const int t8 = lane & 7;
            for (int jb = j_begin; jb < j_end; jb += 2 * n_teams) {
                const int j0 = jb + team;
                const int j1 = j0 + n_teams;
                const bool p0_in = j0 < j_end, p1_in = j1 < j_end;
                // Lanes past the end or without a vector read row 0 and drop the
                // result: every load below is unconditional, no lane-dependent branch.
                // (j0, j1 stay inside the arrays: they are below j_end + 2 * n_teams.)
                int2 s0 = slots[j0], s1 = slots[j1];
                if constexpr (!Layout::kPacked) {
                    s0.y = static_cast<int32_t>(__ldg(L.mapping + (p0_in ? s0.x : 0)));
                    s1.y = static_cast<int32_t>(__ldg(L.mapping + (p1_in ? s1.x : 0)));
                    slots[(t8 == 0 && p0_in) ? j0 : kSpare + lane].y = s0.y;
                    slots[(t8 == 0 && p1_in) ? j1 : kSpare + lane].y = s1.y;
                }
                const bool p0 = p0_in && s0.y >= 0, p1 = p1_in && s1.y >= 0;
                const float *r0 = L.storage + static_cast<int64_t>(p0 ? s0.y : 0) * d;
                const float *r1 = L.storage + static_cast<int64_t>(p1 ? s1.y : 0) * d;
                float a0 = 0.0f, a1 = 0.0f;
                for (int o = 4 * t8; o < d; o += 128) {
                    // up to four stripes of each row in flight before any arithmetic
                    float4 x0[4], x1[4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const bool in = o + 32 * m < d;
                        x0[m] = in ? __ldg(reinterpret_cast<const float4 *>(r0 + o + 32 * m))
                                   : make_float4(0, 0, 0, 0);
                        x1[m] = in ? __ldg(reinterpret_cast<const float4 *>(r1 + o + 32 * m))
                                   : make_float4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        if (o + 32 * m < d) {
                            const float4 qa = *reinterpret_cast<const float4 *>(q_s + o + 32 * m);
                            a0 = stripe(a0, qa, x0[m]);
                            a1 = stripe(a1, qa, x1[m]);
                        }
                    }
                }
                a0 = team_reduce(a0);
                a1 = team_reduce(a1);
                // +inf marks a candidate without a vector: it is never inserted
                cand_d[(t8 == 0 && p0_in) ? j0 : kSpare + lane] = p0 ? a0 : CUDART_INF_F;
                cand_d[(t8 == 0 && p1_in) ? j1 : kSpare + lane] = p1 ? a1 : CUDART_INF_F;
            }
        };
        const int count = deal_count(n_work, beam);  // length of this group's beam list

        if constexpr (CH == 1) {
            // Heap inserts (:206-220): candidate j -> beam (j / 4) mod 4, ascending j;
            // each group walks its beam's list, skipping the candidates its heap
            // would turn down, so that a step of the warp is an operation that changes
            // a heap.  A beam's list has at most 32 candidates: it is kept in
            // registers (lane g: positions g, g + 8, g + 16, g + 24), and the next
            // path is read while the next candidate is being chosen.
            // The first 32 candidates are exactly positions 0-7 of the four lists.
            // All warps evaluate those; then the open warp starts on them while the
            // other three warps evaluate the rest (named barrier 2: 96 threads arrive,
            // the open warp waits when it has used up positions 0-7), and the result
            // warp inserts once everything is known (named barrier 3 among those
            // three warps).  Both barriers complete once per round, and a warp cannot
            // reach the next round's use before the CTA-wide barriers in between.
            constexpr int kFirst = 2 * kBeams * kTeamsPerWarp;  // 32
            distances(w * kTeamsPerWarp + (lane >> 3), kBeams * kTeamsPerWarp, 0,
                      min(n_work, kFirst));
            __syncthreads();
            const bool more = n_work > kFirst;  // uniform over the CTA
            if (w != 0 && more) {
                distances((w - 1) * kTeamsPerWarp + (lane >> 3), (kBeams - 1) * kTeamsPerWarp,
                          kFirst, n_work);
                __threadfence_block();
                asm volatile("bar.arrive 2, 128;" ::: "memory");  // to the open warp
                if (w == 1) asm volatile("bar.sync 3, 96;" ::: "memory");  // result warp waits
                else asm volatile("bar.arrive 3, 96;" ::: "memory");       // for the other two
            }
            if (w < 2) {
                float cd[4];
                auto load_list = [&](int k_from) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int pos = 8 * k + static_cast<int>(gc.g);
                        if (k >= k_from) {  // compile-time after unrolling
                            const float dist = cand_d[deal_index(pos, beam)];  // in bounds
                            cd[k] = pos < count ? dist : CUDART_INF_F;
                        }
                    }
                };
                unsigned ahead = 0xffffffffu;  // positions not yet passed
                if (w == 0) {
                    unsigned leaf = follow_bits<H, W>(o_lb);
                    auto run = [&]() {
                        for (;;) {
                            const ReplacePath<int2> path =
                                replace_load<H, int2>(okey, oval, gc, leaf);
                            const unsigned m = below_mask(cd, path.limit, gc) & ahead;
                            const bool found = m != 0;
                            if (!__any_sync(kFull, found)) break;
                            const unsigned pos = found ? __ffs(m) - 1 : 0u;
                            const float key = list_at(cd, pos);
                            replace_apply<H, W>(okey, oval, o_sb, o_lb, gc, leaf, path, found, key,
                                                slots[deal_index(pos, beam)]);
                            if (found) ahead = 0xfffffffeu << pos;
                            leaf = follow_bits<H, W>(o_lb);
                        }
                    };
                    load_list(0);
                    if (more) {
                        cd[1] = cd[2] = cd[3] = CUDART_INF_F;  // not evaluated yet
                        run();
                        asm volatile("bar.sync 2, 128;" ::: "memory");
                        load_list(1);
                    }
                    run();
                    int valid = 0;
                    for (int jb = 0; jb < n_work; jb += 32)  // slots[jb + lane] is in bounds
                        valid += (jb + lane < n_work) & (slots[jb + lane].y >= 0);
                    n_eval += __reduce_add_sync(kFull, valid);
                } else {
                    load_list(0);
                    for (;;) {
                        const SinkPath<int32_t> path = sink_load<H, W, int32_t>(rkey, rid, r_sb, gc);
                        const unsigned m = below_mask(cd, -r_root, gc) & ahead;
                        const bool found = m != 0;
                        if (!__any_sync(kFull, found)) break;
                        const unsigned pos = found ? __ffs(m) - 1 : 0u;
                        const float key = list_at(cd, pos);
                        const float root = sink_apply<H, W, false>(
                            rkey, rid, r_sb, r_sb, gc, path, found, -key,
                            slots[deal_index(pos, beam)].x);
                        if (found) { r_root = root; ahead = 0xfffffffeu << pos; }
                    }
                }
                pair_sync();  // result roots visible to the open warp before it pops
            }
        } else {
            distances(w * kTeamsPerWarp + (lane >> 3), kBeams * kTeamsPerWarp, 0, n_work);
            __syncthreads();
            if (w < 2) {
                int s = 0;
                if (w == 0) {
                    int valid = 0;
                    for (int j = lane; j < n_work; j += 32) valid += slots[j].y >= 0;
                    n_eval += __reduce_add_sync(kFull, valid);
                    unsigned leaf = follow_bits<H, W>(o_lb);
                    float limit = okey[leaf - 1];
                    for (;;) {
                        s = next_below(cand_d, gc, beam, s, count, limit);
                        const bool found = s < count;
                        if (!__any_sync(kFull, found)) break;
                        const int j = found ? deal_index(s, beam) : 0;
                        group_replace_at<H, W>(okey, oval, o_sb, o_lb, gc, leaf, found, cand_d[j],
                                               slots[j]);
                        s += found;
                        leaf = follow_bits<H, W>(o_lb);
                        limit = okey[leaf - 1];
                    }
                } else {
                    for (;;) {
                        s = next_below(cand_d, gc, beam, s, count, -r_root);
                        const bool found = s < count;
                        if (!__any_sync(kFull, found)) break;
                        const int j = found ? deal_index(s, beam) : 0;
                        const float root = group_sink<H, W, false>(rkey, rid, r_sb, r_sb, gc, found,
                                                                   -cand_d[j], slots[j].x);
                        if (found) { r_root = root; ++s; }
                    }
                }
                pair_sync();  // result roots visible to the open warp before it pops
            }
        }
    }
    __syncthreads();

    // ---- store (:230-245): per beam worst -> best ----------------------------------
    // The result warp pops into the rows of the open heaps' values, which are dead
    // by now; all threads then write the output with coalesced stores.
    const int n_discard = max(H - ef, 0), n_real = min(ef, H);
    if (w == 1) {
        for (int p = 0; p < n_discard + n_real; ++p) {
            const float key = rkey[0];
            const int32_t id = rid[0];
            group_sink<H, W, false>(rkey, rid, r_sb, r_sb, gc, true, CUDART_INF_F, int32_t(-1));
            const int i = p - n_discard;
            oval[(i >= 0 && gc.g == 0) ? i : H + static_cast<int>(gc.g)] =
                make_int2(id, __float_as_int(-key));
        }
    }
    __syncthreads();
    {
        int64_t *oI = out_I + b * kBeams * ef;
        float *oD = out_D + b * kBeams * ef;
        for (int i = threadIdx.x; i < kBeams * n_real; i += kThreads) {
            const int bm = i / n_real, j = i - bm * n_real;
            const int2 e = open_val[bm][j];
            oI[bm * ef + j] = e.x;
            oD[bm * ef + j] = __int_as_float(e.y);
        }
        // ef > H: the heap is exhausted, upstream keeps popping (-1, key +inf)
        const int n_tail = ef - n_real;
        for (int i = threadIdx.x; i < kBeams * n_tail; i += kThreads) {
            const int bm = i / n_tail, j = n_real + (i - bm * n_tail);
            oI[bm * ef + j] = -1;
            oD[bm * ef + j] = -CUDART_INF_F;
        }
    }
    if (stats != nullptr) {
        __syncthreads();
        int bits = 0;
        for (int i = threadIdx.x; i < kBloomWords; i += kThreads) bits += __popc(bloom[i]);
        for (int o = 16; o > 0; o >>= 1) bits += __shfl_down_sync(kFull, bits, o);
        if (lane == 0) {
            atomicAdd(&stat_s[3], bits);
            if (w == 0) { stat_s[0] = n_rounds; stat_s[1] = n_expand; stat_s[2] = n_eval; }
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
#define PA_LAUNCH(HS, CHS)                                                  \
    traverse_kernel<HS, CHS, Layout><<<grid, block, dyn, stream>>>(         \
        L, out_I, out_D, query, init_I, init_D, d, ldq, n_init, ef, stats)
#define PA_LAUNCH_H(HS)                                                     \
    do {                                                                    \
        if (n_nb == 32) PA_LAUNCH(HS, 1);                                   \
        else PA_LAUNCH(HS, 2);                                              \
    } while (0)
    switch (pa_heap_size_for(ef)) {
        case 32: PA_LAUNCH_H(32); break;
        case 64: PA_LAUNCH_H(64); break;
        case 128: PA_LAUNCH_H(128); break;
        default: PA_LAUNCH_H(256); break;
    }
#undef PA_LAUNCH_H
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
    PA_REQUIRE(d <= 4096, "d_model too large for the shared-memory query");
    PA_REQUIRE(n_init >= 0, "n_initials must not be negative");
    PA_REQUIRE(n_nodes >= 0 && n_nodes < 0x7fffffff, "node ids must fit int32");
    if (batch == 0) return PA_OK;
    PA_REQUIRE(out_I && out_D && storage && query, "null pointer");
    PA_REQUIRE(n_init == 0 || (init_I && init_D), "null entry pointer");
    PA_REQUIRE(aligned16(storage) && aligned16(query), "storage / query must be 16-byte aligned");
    return PA_OK;
}

// Every argument check of the packed-layout search, without launching anything.
int traverse_packed_check(const int64_t *output_I, const float *output_D,
                          const int32_t *packed_nbr, const int32_t *row_of, const float *storage,
                          const float *query, int64_t ldq, const int64_t *initial_I,
                          const float *initial_D, int64_t batch, int64_t n_nodes, int d_model,
                          int n_neighbors, int n_initials, int ef_search) {
    int rc = check_common(output_I, output_D, storage, query, initial_I, initial_D, batch, n_nodes,
                          d_model, n_neighbors, n_initials, ef_search);
    if (rc != PA_OK || batch == 0) return rc;
    PA_REQUIRE(packed_nbr && row_of, "null packed-index pointer");
    PA_REQUIRE((reinterpret_cast<uintptr_t>(packed_nbr) & 15u) == 0,
               "packed_nbr must be 16-byte aligned");
    PA_REQUIRE(ldq >= d_model && ldq % 4 == 0, "query row stride must be a multiple of 4");
    return PA_OK;
}

int traverse_packed_launch(int64_t *output_I, float *output_D, const int32_t *packed_nbr,
                           const int32_t *row_of, const float *storage, const float *query,
                           int64_t ldq, const int64_t *initial_I, const float *initial_D,
                           int64_t batch, int64_t n_nodes, int64_t n_storage, int d_model,
                           int n_neighbors, int n_initials, int ef_search, int32_t *stats,
                           cudaStream_t stream) {
    (void)n_storage;
    int rc = traverse_packed_check(output_I, output_D, packed_nbr, row_of, storage, query, ldq,
                                   initial_I, initial_D, batch, n_nodes, d_model, n_neighbors,
                                   n_initials, ef_search);
    if (rc != PA_OK || batch == 0) return rc;
    PackedLayout L{reinterpret_cast<const int4 *>(packed_nbr), row_of, storage, n_nodes};
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

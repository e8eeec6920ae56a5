// Entry routing (FES): nearest router per query, squared distances to that
// router's leaves, and the leaf-id gather.  Replaces upstream
// extension/routing_cuda.cu:10-113 and pilot_ann/layers/entry.py:81-88.
//
// Router choice: squared distances accumulated in double precision in index
// order (acc = acc + diff * diff, each operation rounded), so the chosen router
// is the one exact arithmetic on the float inputs would give; ties go to the
// lowest index.  Leaf distances: upstream's fp32 order -- per 32-wide slice of
// the dimensions a running r = fma(q - p, q - p, r), the slice sums added in
// order to a total that starts at zero.
//
// One CTA per query.  Warp 0..: routers are spread over all threads, the
// winner is reduced through shared memory; then each thread owns one leaf.
#include "pa_common.cuh"

namespace pa {

constexpr int kRouteThreads = 128;

__global__ void __launch_bounds__(kRouteThreads)
route_kernel(int64_t *__restrict__ router, float *__restrict__ leaf_D,
             int64_t *__restrict__ leaf_I, const float *__restrict__ query,
             const float *__restrict__ route_vectors, const int64_t *__restrict__ entry_nodes,
             const float *__restrict__ entry_vectors, int d, int64_t ldq, int n_routers,
             int n_leaves) {
    extern __shared__ __align__(16) float q_s[];
    __shared__ double best_d[kRouteThreads];
    __shared__ int best_r[kRouteThreads];
    const int64_t b = blockIdx.x;
    const int tid = threadIdx.x;
    for (int i = tid; i < d; i += kRouteThreads) q_s[i] = query[b * ldq + i];
    __syncthreads();

    // nearest router (route_vectors == nullptr: a single implicit router)
    double mine = CUDART_INF;
    int mine_r = 0x7fffffff;
    if (route_vectors != nullptr) {
        for (int r = tid; r < n_routers; r += kRouteThreads) {
            const float *p = route_vectors + static_cast<int64_t>(r) * d;
            double acc = 0.0;
            for (int k = 0; k < d; k += 4) {
                float4 pv = __ldg(reinterpret_cast<const float4 *>(p + k));
                float4 qv = *reinterpret_cast<const float4 *>(q_s + k);
                double d0 = __dsub_rn(double(qv.x), double(pv.x));
                double d1 = __dsub_rn(double(qv.y), double(pv.y));
                double d2 = __dsub_rn(double(qv.z), double(pv.z));
                double d3 = __dsub_rn(double(qv.w), double(pv.w));
                acc = __dadd_rn(acc, __dmul_rn(d0, d0));
                acc = __dadd_rn(acc, __dmul_rn(d1, d1));
                acc = __dadd_rn(acc, __dmul_rn(d2, d2));
                acc = __dadd_rn(acc, __dmul_rn(d3, d3));
            }
            if (acc < mine) { mine = acc; mine_r = r; }  // ascending r: first minimum
        }
    } else if (tid == 0) {
        mine = 0.0;
        mine_r = 0;
    }
    best_d[tid] = mine;
    best_r[tid] = mine_r;
    __syncthreads();
    for (int off = kRouteThreads / 2; off > 0; off >>= 1) {
        if (tid < off) {
            double od = best_d[tid + off];
            int orr = best_r[tid + off];
            if (od < best_d[tid] || (od == best_d[tid] && orr < best_r[tid])) {
                best_d[tid] = od;
                best_r[tid] = orr;
            }
        }
        __syncthreads();
    }
    const int r = best_r[0];
    if (tid == 0 && router != nullptr) router[b] = r;

    // leaves of the chosen router
    for (int l = tid; l < n_leaves; l += kRouteThreads) {
        const float *p = entry_vectors + (static_cast<int64_t>(r) * n_leaves + l) * d;
        float total = 0.0f;
        for (int k0 = 0; k0 < d; k0 += 32) {
            float acc = 0.0f;
            const int k1 = min(k0 + 32, d);
            for (int k = k0; k < k1; k += 4) {
                float4 pv = __ldg(reinterpret_cast<const float4 *>(p + k));
                float4 qv = *reinterpret_cast<const float4 *>(q_s + k);
                float d0 = __fsub_rn(qv.x, pv.x), d1 = __fsub_rn(qv.y, pv.y);
                float d2 = __fsub_rn(qv.z, pv.z), d3 = __fsub_rn(qv.w, pv.w);
                acc = __fmaf_rn(d0, d0, acc);
                acc = __fmaf_rn(d1, d1, acc);
                acc = __fmaf_rn(d2, d2, acc);
                acc = __fmaf_rn(d3, d3, acc);
            }
            total = __fadd_rn(total, acc);
        }
        leaf_D[b * n_leaves + l] = total;
        if (leaf_I != nullptr)
            leaf_I[b * n_leaves + l] = __ldg(entry_nodes + static_cast<int64_t>(r) * n_leaves + l);
    }
}

int route_launch(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
                 int64_t ldq, const float *route_vectors, const int64_t *entry_nodes,
                 const float *entry_vectors, int64_t batch, int d, int n_routers, int n_leaves,
                 cudaStream_t stream) {
    if (batch == 0) return PA_OK;
    route_kernel<<<static_cast<unsigned>(batch), kRouteThreads, sizeof(float) * d, stream>>>(
        router, leaf_D, leaf_I, query, route_vectors, entry_nodes, entry_vectors, d, ldq,
        n_routers, n_leaves);
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

}  // namespace pa

extern "C" int pa_route(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
                        const float *route_vectors, const int64_t *entry_nodes,
                        const float *entry_vectors, int64_t batch, int d_model, int n_routers,
                        int n_leaves, void *stream) {
    using namespace pa;
    PA_REQUIRE(batch >= 0 && batch <= 0x7fffffff, "batch out of range");
    PA_REQUIRE(n_leaves > 0 && n_leaves % 32 == 0, "n_leaves must be a multiple of 32");
    PA_REQUIRE(n_routers > 0, "n_routers must be positive");
    PA_REQUIRE(d_model > 0 && d_model % 4 == 0 && d_model <= 8192,
               "d_model must be a multiple of 4 (at most 8192)");
    if (batch == 0) return PA_OK;
    PA_REQUIRE(leaf_D && query && entry_vectors, "null pointer");
    PA_REQUIRE(leaf_I == nullptr || entry_nodes != nullptr, "leaf_I needs entry_nodes");
    PA_REQUIRE(route_vectors != nullptr || n_routers == 1, "route_vectors missing");
    PA_REQUIRE(aligned16(query) && aligned16(entry_vectors) &&
                   (route_vectors == nullptr || aligned16(route_vectors)),
               "vectors must be 16-byte aligned");
    return route_launch(router, leaf_D, leaf_I, query, d_model, route_vectors, entry_nodes,
                        entry_vectors, batch, d_model, n_routers, n_leaves, static_cast<cudaStream_t>(stream));
}

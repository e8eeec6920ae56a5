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
// The dense part -- every query against every router -- is a contraction and
// runs on the tensor cores when the caller supplies workspace: q.r for all pairs
// by the tcgen05 GEMM of project.cu (fp32-grade, three TF32 products), then
// score(r) = |r|^2 - 2 q.r.  The tensor-core scores only shortlist: every router
// whose score is within a conservative margin of the best one is re-measured
// exactly (the double-precision sum above), so the id that comes out is the exact
// one in either mode; normally the shortlist holds a single router.
//
// One CTA per query: shortlist + exact re-measure, the winner reduced through
// shared memory; then each thread owns one leaf.
#include "pa_common.cuh"

namespace pa {

constexpr int kRouteThreads = 128;

__global__ void __launch_bounds__(kRouteThreads)
route_kernel(int64_t *__restrict__ router, float *__restrict__ leaf_D,
             int64_t *__restrict__ leaf_I, const float *__restrict__ query,
             const float *__restrict__ route_vectors, const int64_t *__restrict__ entry_nodes,
             const float *__restrict__ entry_vectors, int d, int64_t ldq, int n_routers,
             int n_leaves, const float *__restrict__ dots, const float *__restrict__ rnorm2,
             const int *__restrict__ gemm_status) {
    extern __shared__ __align__(16) float q_s[];
    __shared__ double best_d[kRouteThreads];
    __shared__ int best_r[kRouteThreads];
    const int64_t b = blockIdx.x;
    const int tid = threadIdx.x;
    for (int i = tid; i < d; i += kRouteThreads) q_s[i] = query[b * ldq + i];
    __syncthreads();

    // tensor-core scores: shortlist the routers within `margin` of the best score.
    // margin >> the error of a score (a few 1e-6 * |q||r|), so the exact winner and
    // everything tied with it are always on the list.
    float cutoff = CUDART_INF_F;
    // a tensor-core GEMM that gave up on a bounded wait leaves `dots` unwritten
    if (dots != nullptr && gemm_status != nullptr && *gemm_status != 0) dots = nullptr;
    if (dots != nullptr) {
        __shared__ float red_a[kRouteThreads], red_b[kRouteThreads], red_c[kRouteThreads];
        float best = CUDART_INF_F, rmax = 0.0f, qn = 0.0f;
        for (int r = tid; r < n_routers; r += kRouteThreads) {
            const float n2 = rnorm2[r];
            best = fminf(best, n2 - 2.0f * dots[b * n_routers + r]);
            rmax = fmaxf(rmax, n2);
        }
        for (int k = tid; k < d; k += kRouteThreads) qn += q_s[k] * q_s[k];
        red_a[tid] = best; red_b[tid] = rmax; red_c[tid] = qn;
        __syncthreads();
        for (int off = kRouteThreads / 2; off > 0; off >>= 1) {
            if (tid < off) {
                red_a[tid] = fminf(red_a[tid], red_a[tid + off]);
                red_b[tid] = fmaxf(red_b[tid], red_b[tid + off]);
                red_c[tid] += red_c[tid + off];
            }
            __syncthreads();
        }
        cutoff = red_a[0] + 1e-4f * (red_b[0] + red_c[0]);
    }

    // nearest router (route_vectors == nullptr: a single implicit router).  Pass 0
    // measures the shortlist (every router without tensor-core scores); pass 1
    // runs only when pass 0 chose nothing -- the scores were unusable (NaN / Inf
    // in the query, or a GEMM that gave up) -- and measures every router.
    int r = 0;
    for (int pass = 0; pass < 2; ++pass) {
        const bool listed = pass == 0 && dots != nullptr;
        double mine = CUDART_INF;
        int mine_r = 0x7fffffff;
        if (route_vectors != nullptr) {
            for (int rr = tid; rr < n_routers; rr += kRouteThreads) {
                if (listed && !(rnorm2[rr] - 2.0f * dots[b * n_routers + rr] <= cutoff))
                    continue;  // not on the shortlist
                const float *p = route_vectors + static_cast<int64_t>(rr) * d;
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
                if (acc < mine) { mine = acc; mine_r = rr; }  // ascending rr: first minimum
            }
        } else if (tid == 0) {
            mine = 0.0;
            mine_r = 0;
        }
        __syncthreads();  // the previous pass has read best_r[0]
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
        r = best_r[0];
        if (static_cast<unsigned>(r) < static_cast<unsigned>(n_routers) || !listed) break;
    }
    // No distance compared below +inf (a NaN or Inf query): upstream's argmin still
    // returns an index in range; router 0 here.  r indexes device memory below.
    if (static_cast<unsigned>(r) >= static_cast<unsigned>(n_routers)) r = 0;
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

__global__ void router_norms_kernel(float *__restrict__ rnorm2,
                                    const float *__restrict__ route_vectors, int n_routers, int d) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= n_routers) return;
    float acc = 0.0f;
    for (int k = lane; k < d; k += 32) {
        const float x = route_vectors[static_cast<int64_t>(r) * d + k];
        acc += x * x;
    }
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
    if (lane == 0) rnorm2[r] = acc;
}

int router_norms_launch(float *rnorm2, const float *route_vectors, int n_routers, int d,
                        cudaStream_t stream) {
    router_norms_kernel<<<(n_routers + 3) / 4, 128, 0, stream>>>(rnorm2, route_vectors, n_routers, d);
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

// dots_ws: nullptr, or room for batch * n_routers floats; rnorm2: |r|^2 per router
// (router_norms_launch).  Without workspace every router is measured exactly.
int route_launch(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
                 int64_t ldq, const float *route_vectors, const int64_t *entry_nodes,
                 const float *entry_vectors, int64_t batch, int d, int n_routers, int n_leaves,
                 float *dots_ws, const float *rnorm2, cudaStream_t stream) {
    if (batch == 0) return PA_OK;
    const bool tensor = dots_ws != nullptr && rnorm2 != nullptr && route_vectors != nullptr &&
                        n_routers > 1 && d % 4 == 0 && ldq % 4 == 0;
    if (tensor) {
        int rc = gemm_tf32x3_launch(dots_ws, query, route_vectors, static_cast<int>(batch),
                                    n_routers, d, ldq, d, n_routers, stream);
        if (rc != PA_OK) return rc;
    }
    route_kernel<<<static_cast<unsigned>(batch), kRouteThreads, sizeof(float) * d, stream>>>(
        router, leaf_D, leaf_I, query, route_vectors, entry_nodes, entry_vectors, d, ldq,
        n_routers, n_leaves, tensor ? dots_ws : nullptr, tensor ? rnorm2 : nullptr,
        tensor ? gemm_status_address() : nullptr);
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
    // without workspace every router is measured exactly on the CUDA cores; the
    // tensor-core shortlist needs pa_route_ws
    return route_launch(router, leaf_D, leaf_I, query, d_model, route_vectors, entry_nodes,
                        entry_vectors, batch, d_model, n_routers, n_leaves, nullptr, nullptr,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int64_t pa_route_workspace_floats(int64_t batch, int n_routers) {
    return (batch + 1) * static_cast<int64_t>(n_routers);
}

extern "C" int pa_route_ws(int64_t *router, float *leaf_D, int64_t *leaf_I, const float *query,
                           const float *route_vectors, const int64_t *entry_nodes,
                           const float *entry_vectors, int64_t batch, int d_model, int n_routers,
                           int n_leaves, float *workspace, void *stream) {
    using namespace pa;
    if (workspace == nullptr || route_vectors == nullptr || n_routers <= 1 || batch <= 0)
        return pa_route(router, leaf_D, leaf_I, query, route_vectors, entry_nodes, entry_vectors,
                        batch, d_model, n_routers, n_leaves, stream);
    PA_REQUIRE(batch <= 0x7fffffff, "batch out of range");
    PA_REQUIRE(n_leaves > 0 && n_leaves % 32 == 0, "n_leaves must be a multiple of 32");
    PA_REQUIRE(d_model > 0 && d_model % 4 == 0 && d_model <= 8192,
               "d_model must be a multiple of 4 (at most 8192)");
    PA_REQUIRE(leaf_D && query && entry_vectors, "null pointer");
    PA_REQUIRE(leaf_I == nullptr || entry_nodes != nullptr, "leaf_I needs entry_nodes");
    PA_REQUIRE(aligned16(query) && aligned16(entry_vectors) && aligned16(route_vectors) &&
                   aligned16(workspace),
               "vectors and workspace must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *rnorm2 = workspace + batch * n_routers;
    int rc = router_norms_launch(rnorm2, route_vectors, n_routers, d_model, st);
    if (rc != PA_OK) return rc;
    return route_launch(router, leaf_D, leaf_I, query, d_model, route_vectors, entry_nodes,
                        entry_vectors, batch, d_model, n_routers, n_leaves, workspace, rnorm2, st);
}

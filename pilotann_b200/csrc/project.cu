// Query projection: rotated = query @ VT^T (upstream runs this on the CPU,
// pilot_ann/layers/staged.py:198).  out[b, j] = sum_k query[b, k] * VT[j, k].
// Both operands are K-major, the natural "TN" contraction.
#include "pa_common.cuh"

namespace pa {

constexpr int kPT = 64;   // output tile (queries x columns)
constexpr int kPK = 16;   // k slice

// fp32 CUDA-core path: 16x16 threads, each a 4x4 micro-tile, fma in k order.
__global__ void __launch_bounds__(256)
project_kernel(float *__restrict__ out, const float *__restrict__ query,
               const float *__restrict__ VT, int64_t batch, int d, int d_out, int64_t ld_out) {
    __shared__ float q_s[kPK][kPT + 4];
    __shared__ float v_s[kPK][kPT + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t b0 = blockIdx.y * static_cast<int64_t>(kPT);
    const int j0 = blockIdx.x * kPT;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < d; k0 += kPK) {
        for (int i = threadIdx.x; i < kPT * kPK; i += 256) {
            int r = i / kPK, k = i % kPK;
            int64_t bb = b0 + r;
            int jj = j0 + r;
            q_s[k][r] = (bb < batch && k0 + k < d) ? query[bb * d + k0 + k] : 0.0f;
            v_s[k][r] = (jj < d_out && k0 + k < d) ? VT[static_cast<int64_t>(jj) * d + k0 + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kPK; ++k) {
            float a[4], c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = q_s[k][ty * 4 + i]; c[i] = v_s[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(a[i], c[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t bb = b0 + ty * 4 + i;
        if (bb >= batch) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int jj = j0 + tx * 4 + j;
            if (jj < d_out) out[bb * ld_out + jj] = acc[i][j];
        }
    }
}

int project_launch(float *out, const float *query, const float *VT, int64_t batch, int d,
                   int d_out, int64_t ld_out, cudaStream_t stream) {
    if (batch == 0 || d_out == 0) return PA_OK;
    dim3 grid((d_out + kPT - 1) / kPT, static_cast<unsigned>((batch + kPT - 1) / kPT));
    project_kernel<<<grid, 256, 0, stream>>>(out, query, VT, batch, d, d_out, ld_out);
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

}  // namespace pa

extern "C" int pa_project(float *out, const float *query, const float *VT, int64_t batch,
                          int d_model, int d_out, int64_t ld_out, void *stream) {
    using namespace pa;
    PA_REQUIRE(batch >= 0 && batch <= 0x7fffffff, "batch out of range");
    PA_REQUIRE(d_model > 0 && d_out >= 0 && ld_out >= d_out, "bad projection sizes");
    if (batch == 0 || d_out == 0) return PA_OK;
    PA_REQUIRE(out && query && VT, "null pointer");
    return project_launch(out, query, VT, batch, d_model, d_out, ld_out,
                          static_cast<cudaStream_t>(stream));
}

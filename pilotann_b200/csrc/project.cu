// Query projection: rotated = query @ VT^T (upstream runs this on the CPU,
// pilot_ann/layers/staged.py:198).  out[b, j] = sum_k query[b, k] * VT[j, k].
// Both operands are K-major, the natural "TN" contraction.
#include <cuda.h>

#include "pa_common.cuh"
#include "tc05.cuh"

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

// ---- tensor-core path (TMA -> shared memory -> tcgen05, TMEM accumulator) ------
// out[m, n] = sum_k A[m, k] * B[n, k]; A, B fp32, both K-major.  fp32-grade
// accuracy from TF32 tensor cores by the three-product split: x = big + small
// with big = x truncated to TF32 and small = x - big (exact in fp32);
// A.B ~= Asmall.Bbig + Abig.Bsmall + Abig.Bbig, all accumulated in one fp32 TMEM
// tile.
//
// CTA tile 128 x 64, K slice 32 floats (one 128-byte swizzle row = four K=8 MMA
// steps), four stages, warp-specialised: a control thread keeps bulk-tensor
// (TMA) copies of the raw A and B tiles three slices ahead (SWIZZLE_128B,
// out-of-range rows and columns zero-filled, completion on the stage's "full"
// mbarrier); eight converter warps split each raw tile in place (raw -> big,
// small to a second buffer; the transform is element-wise, so the swizzled
// layout is untouched) and arrive on the stage's "converted" mbarrier; the control
// thread then issues the 12 MMAs of the slice and commits them to the stage's
// "empty" mbarrier, after which the stage may be refilled.  No CTA-wide barrier
// inside the K loop.  Epilogue: warps 0-3 read their 32 TMEM lanes with
// tcgen05.ld and store rows.  Every wait is bounded.
namespace gemm {
constexpr int BM = 128, BN = 64, BK = 32, STAGES = 4;
constexpr int CONVERTERS = 256;           // threads that split the raw tiles
constexpr int THREADS = CONVERTERS + 32;  // + one warp whose lane 0 drives TMA and MMA
constexpr int A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4;
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr int DYN_SMEM = STAGES * STAGE_BYTES + 1024;
constexpr uint32_t WAIT_LIMIT = 1u << 20;
}  // namespace gemm

__device__ int g_gemm_status = 0;  // 1 = a bounded wait ran out

// raw fp32 chunk at `big_addr` -> TF32-exact part in place, remainder to `small_addr`
__device__ __forceinline__ void split_in_place(uint32_t big_addr, uint32_t small_addr) {
    float4 x, b, s;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w) : "r"(big_addr) : "memory");
    b.x = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u);
    b.y = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u);
    b.z = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u);
    b.w = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u);
    s.x = __fsub_rn(x.x, b.x); s.y = __fsub_rn(x.y, b.y);
    s.z = __fsub_rn(x.z, b.z); s.w = __fsub_rn(x.w, b.w);
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(big_addr), "f"(b.x), "f"(b.y),
                 "f"(b.z), "f"(b.w) : "memory");
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(small_addr), "f"(s.x), "f"(s.y),
                 "f"(s.z), "f"(s.w) : "memory");
}

__global__ void __launch_bounds__(gemm::THREADS, 1)
gemm_tf32x3_kernel(float *__restrict__ out, const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b, int M, int N, int K, int64_t ldo) {
    using namespace gemm;
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], conv_bar[STAGES], empty_bar[STAGES];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_s;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t tiles = (tc05::smem_u32(dyn_smem) + 1023u) & ~1023u;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nkb = (K + BK - 1) / BK;

    auto stage_a = [&](int s) { return tiles + s * STAGE_BYTES; };
    auto stage_b = [&](int s) { return tiles + s * STAGE_BYTES + 2 * A_BYTES; };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc05::mbar_init(tc05::smem_u32(&full_bar[s]), 1);
            tc05::mbar_init(tc05::smem_u32(&conv_bar[s]), CONVERTERS / 32);
            tc05::mbar_init(tc05::smem_u32(&empty_bar[s]), 1);
        }
        abort_s = 0;
        tc05::fence_barrier_init();
    }
    if (warp == 0) tc05::tmem_alloc(tc05::smem_u32(&tmem_slot), BN);
    tc05::fence_before_sync();
    __syncthreads();
    tc05::fence_after_sync();
    const uint32_t tmem = tmem_slot;
    constexpr uint32_t idesc = tc05::idesc_tf32(BM, BN);

    if (tid == CONVERTERS) {
        // ---- control thread: TMA producer and MMA issuer -----------------------
        tc05::tma_prefetch_desc(&map_a);
        tc05::tma_prefetch_desc(&map_b);
        auto fill = [&](int kb) {  // raw tiles of slice kb into its stage
            const int s = kb % STAGES;
            const uint32_t bar = tc05::smem_u32(&full_bar[s]);
            tc05::mbar_expect_tx(bar, A_BYTES + B_BYTES);
            tc05::tma_load_2d(stage_a(s), &map_a, kb * BK, m0, bar);
            tc05::tma_load_2d(stage_b(s), &map_b, kb * BK, n0, bar);
        };
        for (int kb = 0; kb < nkb && kb < STAGES - 1; ++kb) fill(kb);
        for (int kb = 0; kb < nkb && !abort_s; ++kb) {
            const int s = kb % STAGES, use = kb / STAGES;
            // keep the copies STAGES - 1 slices ahead: the stage to refill was read
            // by the MMAs of slice kb - 1
            const int kn = kb + STAGES - 1;
            if (kn < nkb) {
                if (kn >= STAGES &&
                    !tc05::mbar_wait_bounded(tc05::smem_u32(&empty_bar[kn % STAGES]),
                                             ((kn / STAGES) - 1) & 1, WAIT_LIMIT)) {
                    abort_s = 1;
                    break;
                }
                fill(kn);
            }
            if (!tc05::mbar_wait_bounded(tc05::smem_u32(&conv_bar[s]), use & 1, WAIT_LIMIT)) {
                abort_s = 1;
                break;
            }
            tc05::fence_after_sync();
            const uint32_t a_big = stage_a(s), a_small = a_big + A_BYTES;
            const uint32_t b_big = stage_b(s), b_small = b_big + B_BYTES;
#pragma unroll
            for (int k8 = 0; k8 < BK / 8; ++k8) {
                const uint64_t da_b = tc05::smem_desc_sw128(a_big + k8 * 32);
                const uint64_t da_s = tc05::smem_desc_sw128(a_small + k8 * 32);
                const uint64_t db_b = tc05::smem_desc_sw128(b_big + k8 * 32);
                const uint64_t db_s = tc05::smem_desc_sw128(b_small + k8 * 32);
                tc05::mma_tf32(tmem, da_s, db_b, idesc, (kb | k8) != 0);
                tc05::mma_tf32(tmem, da_b, db_s, idesc, 1);
                tc05::mma_tf32(tmem, da_b, db_b, idesc, 1);
            }
            tc05::mma_commit(tc05::smem_u32(&empty_bar[s]));
        }
    } else if (tid < CONVERTERS) {
        // ---- converter warps: raw tile -> (big in place, small) ---------------
        for (int kb = 0; kb < nkb && !abort_s; ++kb) {
            const int s = kb % STAGES, use = kb / STAGES;
            if (!tc05::mbar_wait_bounded(tc05::smem_u32(&full_bar[s]), use & 1, WAIT_LIMIT)) {
                abort_s = 1;
                break;
            }
            const uint32_t a_big = stage_a(s), a_small = a_big + A_BYTES;
            const uint32_t b_big = stage_b(s), b_small = b_big + B_BYTES;
#pragma unroll
            for (int i = 0; i < A_BYTES / 16 / CONVERTERS; ++i) {
                const uint32_t o = (tid + CONVERTERS * i) * 16u;
                split_in_place(a_big + o, a_small + o);
            }
#pragma unroll
            for (int i = 0; i < B_BYTES / 16 / CONVERTERS; ++i) {
                const uint32_t o = (tid + CONVERTERS * i) * 16u;
                split_in_place(b_big + o, b_small + o);
            }
            tc05::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) tc05::mbar_arrive(tc05::smem_u32(&conv_bar[s]));
        }
    }
    // everyone: the last commit covers every MMA issued before it
    bool aborted = abort_s != 0;
    if (nkb > 0 && !aborted) {
        const int last = nkb - 1;
        if (!tc05::mbar_wait_bounded(tc05::smem_u32(&empty_bar[last % STAGES]),
                                     (last / STAGES) & 1, WAIT_LIMIT))
            aborted = true;
    }
    tc05::fence_after_sync();
    if (aborted) {
        if (tid == 0) atomicExch(&g_gemm_status, 1);
    } else if (warp < 4) {
        const int m = m0 + 32 * warp + lane;
        const bool vec = (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            if (nkb > 0) {
                tc05::tmem_ld_32x32(tmem + ((32u * warp) << 16) + c0, r);
                tc05::tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0;
            }
            if (m < M) {
                float *dst = out + m * ldo + n0 + c0;
                if (vec && n0 + c0 + 32 <= N) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4 *>(dst + j) =
                            make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                        __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + c0 + j < N) dst[j] = __uint_as_float(r[j]);
                }
            }
        }
    }
    tc05::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc05::tmem_dealloc(tmem, BN);
}

// Diagnostic: the give-up path of the GEMM, alone.  One thread waits a handful of
// polls on an mbarrier phase that nothing completes, records the failure in the
// status word exactly as the GEMM does, and returns; nothing is left pending.
__global__ void bounded_wait_selftest_kernel(uint32_t polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        tc05::mbar_init(tc05::smem_u32(&bar), 1);
        tc05::fence_barrier_init();
        if (!tc05::mbar_wait_bounded(tc05::smem_u32(&bar), 0, polls)) atomicExch(&g_gemm_status, 1);
    }
}

static bool gemm_operands_ok(const float *A, const float *B, int K, int64_t lda, int64_t ldb) {
    return K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && aligned16(A) && aligned16(B);
}

// cuTensorMapEncodeTiled, looked up through the runtime (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// K-major fp32 matrix [rows, K] with row stride ld, tiles of box_rows x 32 floats
static int make_tile_map(CUtensorMap *map, const float *base, int rows, int K, int64_t ld,
                         int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(PA_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(float)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(gemm::BK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims,
                     strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        return fail(PA_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(rc));
    return PA_OK;
}

// Device address of the status word on the current device (nullptr if the lookup
// fails): kernels that consume a GEMM's output read it to learn that the GEMM gave
// up.  Looked up once per device.
const int *gemm_status_address() {
    static const int *addr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (addr[dev] == nullptr) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_gemm_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        addr[dev] = static_cast<const int *>(p);
    }
    return addr[dev];
}

int gemm_tf32x3_launch(float *out, const float *A, const float *B, int M, int N, int K,
                       int64_t lda, int64_t ldb, int64_t ldo, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    PA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        PA_CUDA_TRY(cudaFuncSetAttribute(gemm_tf32x3_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         gemm::DYN_SMEM));
        configured[dev] = true;
    }
    CUtensorMap map_a, map_b;
    int rc = make_tile_map(&map_a, A, M, K, lda, gemm::BM);
    if (rc != PA_OK) return rc;
    rc = make_tile_map(&map_b, B, N, K, ldb, gemm::BN);
    if (rc != PA_OK) return rc;
    dim3 grid((N + gemm::BN - 1) / gemm::BN, (M + gemm::BM - 1) / gemm::BM);
    gemm_tf32x3_kernel<<<grid, gemm::THREADS, gemm::DYN_SMEM, stream>>>(out, map_a, map_b, M, N, K,
                                                                        ldo);
    count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

int project_launch(float *out, const float *query, const float *VT, int64_t batch, int d,
                   int d_out, int64_t ld_out, cudaStream_t stream) {
    if (batch == 0 || d_out == 0) return PA_OK;
    // tensor cores whenever the operands can be read as aligned float4 rows
    if (gemm_operands_ok(query, VT, d, d, d))
        return gemm_tf32x3_launch(out, query, VT, static_cast<int>(batch), d_out, d, d, d, ld_out,
                                  stream);
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

extern "C" int pa_selftest_bounded_wait(void *stream) {
    pa::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(16u);
    pa::count_launch();
    PA_CUDA_TRY(cudaGetLastError());
    return PA_OK;
}

extern "C" int pa_device_status(int reset) {
    int status = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return PA_ERR_CUDA;
    if (cudaMemcpyFromSymbol(&status, pa::g_gemm_status, sizeof(int)) != cudaSuccess)
        return PA_ERR_CUDA;
    if (reset && status != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(pa::g_gemm_status, &zero, sizeof(int));
    }
    return status;
}

// True 32-bit matrix product for the float32 path: out[n, m] = sum_k x[n, k] * w[m, k].
// IEEE float32 multiply-adds on the CUDA cores: no tensor cores, no TF32, no reduced-precision
// staging.  Every output element is one chain of fused multiply-adds over k = 0, 1, ... K-1 in
// that order, whatever the number of rows and whichever of the two kernels below runs, so a row's
// result does not depend on the batch it is in.
//
// It stands where the reference calls F.linear in float32 with TF32 switched off
// (src/layers/linear.py:19-20, src/distengine/worker.py:427-428).

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int BM = 64;   // rows of x per block
constexpr int BN = 64;   // rows of w (output features) per block
constexpr int BK = 16;

template <bool VEC4>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                int n_rows, int m_cols, int k_dim, int ldx, int ldw, int ldo) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];

    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;

    // each thread stages 4 consecutive k of one row of each tile
    const int l_row = tid / 4, l_k = (tid % 4) * 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    pdl_wait();
    for (int k0 = 0; k0 < k_dim; k0 += BK) {
        float xv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int gr = row0 + l_row, gc = col0 + l_row, gk = k0 + l_k;
        if (gr < n_rows) {
            const float* p = x + (size_t)gr * ldx + gk;
            if (VEC4 && gk + 3 < k_dim) {
                const float4 t = *reinterpret_cast<const float4*>(p);
                xv[0] = t.x; xv[1] = t.y; xv[2] = t.z; xv[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (gk + i < k_dim) xv[i] = p[i];
            }
        }
        if (gc < m_cols) {
            const float* p = w + (size_t)gc * ldw + gk;
            if (VEC4 && gk + 3 < k_dim) {
                const float4 t = *reinterpret_cast<const float4*>(p);
                wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (gk + i < k_dim) wv[i] = p[i];
            }
        }
        __syncthreads();                       // the previous tile has been consumed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            xs[l_k + i][l_row] = xv[i];
            ws[l_k + i][l_row] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx * 4 + j;
            if (c < m_cols) out[(size_t)r * ldo + c] = acc[i][j];
        }
    }
}

// Few rows (decode steps): the same chains of multiply-adds, so the same bits, but tiles of 16
// rows of x by 16 rows of w and a whole slice of k = 64 a stage, so that a product of 8 tokens
// against 2,048 rows of w is 128 blocks that stream w through four stages of cp.async, instead of
// 32 blocks of the wide kernel that each wait for every 16 k.  Thread (ty, tx) owns out[ty][tx]
// and walks k in ascending order, four values a load from shared memory.
constexpr int SM_ROWS = 16, SM_COLS = 16, SM_K = 64, SM_STAGES = 4, SM_LD = SM_K + 4;

__device__ __forceinline__ void cp_async16_f32(void* smem, const void* gmem, bool pred) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

__global__ void __launch_bounds__(SM_ROWS * SM_COLS)
gemm_f32_small_kernel(const float* __restrict__ x, const float* __restrict__ w,
                      float* __restrict__ out, int n_rows, int m_cols, int k_dim, int ldx, int ldw,
                      int ldo) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                                        // [STAGES][ROWS][LD]
    float* ws = smem + SM_STAGES * SM_ROWS * SM_LD;          // [STAGES][COLS][LD]
    const int tid = threadIdx.x;
    const int ty = tid / SM_COLS, tx = tid % SM_COLS;
    const int row0 = blockIdx.y * SM_ROWS, col0 = blockIdx.x * SM_COLS;
    // staging: thread t copies 16 bytes (4 k) of row t / 16 of each tile
    const int l_row = tid / 16, l_k = (tid % 16) * 4;
    const int tiles = (k_dim + SM_K - 1) / SM_K;             // k_dim is a multiple of 4 here

    auto stage_w = [&](int tile, int stage) {
        const int gk = tile * SM_K + l_k, gc = col0 + l_row;
        const bool ok = tile < tiles && gc < m_cols && gk < k_dim;
        cp_async16_f32(ws + (stage * SM_COLS + l_row) * SM_LD + l_k,
                       ok ? w + (size_t)gc * ldw + gk : w, ok);
    };
    auto stage_x = [&](int tile, int stage) {
        const int gk = tile * SM_K + l_k, gr = row0 + l_row;
        const bool ok = tile < tiles && gr < n_rows && gk < k_dim;
        cp_async16_f32(xs + (stage * SM_ROWS + l_row) * SM_LD + l_k,
                       ok ? x + (size_t)gr * ldx + gk : x, ok);
    };
    // the weights do not depend on the kernel before this one: their first stages are requested
    // before the wait
#pragma unroll
    for (int t = 0; t < SM_STAGES - 1; ++t) stage_w(t, t);
    pdl_wait();
#pragma unroll
    for (int t = 0; t < SM_STAGES - 1; ++t) {
        stage_x(t, t);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    float acc = 0.0f;
    for (int tile = 0; tile < tiles; ++tile) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SM_STAGES - 2));
        __syncthreads();                     // this tile has landed; the stage refilled below is free
        const int next = tile + SM_STAGES - 1;
        stage_w(next, next % SM_STAGES);
        stage_x(next, next % SM_STAGES);
        asm volatile("cp.async.commit_group;\n" ::);
        const float* xr = xs + ((tile % SM_STAGES) * SM_ROWS + ty) * SM_LD;
        const float* wr = ws + ((tile % SM_STAGES) * SM_COLS + tx) * SM_LD;
#pragma unroll
        for (int k = 0; k < SM_K; k += 4) {
            const float4 a = *reinterpret_cast<const float4*>(xr + k);
            const float4 b = *reinterpret_cast<const float4*>(wr + k);
            acc = fmaf(a.x, b.x, acc);
            acc = fmaf(a.y, b.y, acc);
            acc = fmaf(a.z, b.z, acc);
            acc = fmaf(a.w, b.w, acc);
        }
    }
    pdl_trigger();
    const int r = row0 + ty, c = col0 + tx;
    if (r < n_rows && c < m_cols) out[(size_t)r * ldo + c] = acc;
}

}  // namespace

DE_EXPORT int de_gemm_f32_small_rows() { return 2 * SM_ROWS; }

DE_EXPORT int de_gemm_f32(const float* x, const float* w, float* out, int n_rows, int m_cols,
                          int k_dim, int ldx, int ldw, int ldo, void* stream) {
    if (n_rows <= 0 || m_cols <= 0) return 0;
    if (k_dim <= 0) return -2;
    dim3 grid((m_cols + BN - 1) / BN, (n_rows + BM - 1) / BM);
    if (grid.y > 65535) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = (ldx % 4 == 0) && (ldw % 4 == 0) && (((uintptr_t)x) % 16 == 0) &&
                     (((uintptr_t)w) % 16 == 0);
    // few rows: the kernel of narrow tiles (zeros beyond k_dim add nothing to a chain, so its
    // results are the wide kernel's, bit for bit)
    if (vec && k_dim % 4 == 0 && n_rows <= 2 * SM_ROWS) {
        const size_t smem = (size_t)SM_STAGES * (SM_ROWS + SM_COLS) * SM_LD * sizeof(float);
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(gemm_f32_small_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        dim3 small((m_cols + SM_COLS - 1) / SM_COLS, (n_rows + SM_ROWS - 1) / SM_ROWS);
        return de_launch(gemm_f32_small_kernel, small, dim3(SM_ROWS * SM_COLS), smem, s, x, w, out,
                         n_rows, m_cols, k_dim, ldx, ldw, ldo);
    }
    if (vec)
        return de_launch(gemm_f32_kernel<true>, grid, dim3(256), 0, s, x, w, out, n_rows, m_cols,
                         k_dim, ldx, ldw, ldo);
    return de_launch(gemm_f32_kernel<false>, grid, dim3(256), 0, s, x, w, out, n_rows, m_cols,
                     k_dim, ldx, ldw, ldo);
}

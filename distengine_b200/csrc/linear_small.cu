// Matrix products for a handful of tokens (decode steps): out[m, n] = sum_k x[m, k] * w[n, k],
// bfloat16 operands, float32 accumulation, for up to 32 rows of x.  Such a product only streams the
// weight matrix once, so the kernel is built around the loads: every thread reads its weight rows in
// 16-byte pieces that a quad of lanes strings together into full 128-byte lines, many in flight per
// thread, straight into tensor-core fragments (no shared-memory staging), and feeds mma.sync
// m16n8k16 with the weights as the 16-row operand and the tokens as the 8-column operand.
//
// Contiguous loads as fragments: lane (g, t) of a warp holds, for a block of 64 k, two pieces of 8
// consecutive elements, k0 + 8 t .. + 7 and k0 + 32 + 8 t .. + 7, of weight rows g and g + 8 and of
// token row g; the four lanes of a quad read 64 contiguous bytes of a row with one instruction.
// Each piece feeds two mma steps (elements 0..3 and 4..7); the k order inside a step is permuted
// against the usual layout, identically for both operands, which a sum over k does not see.
//
// The weights are no kernel's output, so the first blocks of them are requested before the kernel
// waits for the kernel before it in the stream (programmatic dependent launch): the weight stream
// of one product starts while the previous kernel is still finishing.
//
// A block of 8 warps owns 16 (or 8) weight rows; its warps take the 64-wide k blocks in turn and
// their partial sums are added through shared memory.  Optional epilogue: silu(gate) * up, when
// the matrix stacks the gate rows over the up rows ([2 inner, k]); a block then owns 16 gate rows
// and the 16 up rows that belong to them, and writes inner outputs
// (src/layers/activation.py:6-9, src/models/llama.py:23-27).
//
// Stands where the reference calls F.linear (src/layers/linear.py:19-20) on [B, 1, H] inputs.
//
// The RMS norm between two products of a decode layer (src/layers/layernorm.py:12-23,
// src/models/llama.py:74-89) can ride on them instead of being a kernel of its own (`Norm` below).
// The product before the norm adds its (bfloat16-rounded) result to the float32 residual, writes
// residual * norm weight in bfloat16 - the norm's output but for the row's factor
// rsqrt(mean of squares + eps) - and leaves each block's share of every row's sum of squares.  The
// product after the norm multiplies with those rows and applies the row's factor, which is a
// scalar that commutes with the product, to its float32 sums before anything else happens to
// them.  All of it is float32; the shares are added in a fixed order.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int WARPS = 8;
constexpr int KB = 64;                       // k elements per block

__device__ __forceinline__ uint4 load_stream(const void* p) {      // weights: read once
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 load_cached(const void* p) {      // tokens: shared by all blocks
    return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ const unsigned* regs(const uint4& v) {
    return reinterpret_cast<const unsigned*>(&v);
}

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// What the epilogue does for the norms around a product (all pointers may be null).
struct Norm {
    // the norm before this product: x holds rows without their factor; row m's sum of squares is
    // the sum of in_parts[m * in_count + p], p < in_count
    const float* in_parts;
    int in_count;
    float inv_width, eps;
    // the norm after this product: resid[m, n] += result; out[m, n] = resid[m, n] * weight[n];
    // out_parts[m * gridDim.x + blockIdx.x] = the block's share of row m's sum of squares
    float* resid;
    int ld_resid;
    const __nv_bfloat16* weight;
    float* out_parts;
};

// blocks of k that a warp loads before it multiplies any of them: 8 to 16 loads of 16 bytes in
// flight per thread
__host__ __device__ constexpr int blocks_per_round(int nt, int rows, bool gated) {
    const int loads = (gated ? 2 : 1) * (rows == 16 ? 2 : 1) * 2 + nt * 2;
    return 16 / loads > 0 ? 16 / loads : 1;
}

// NT: token tiles of 8 (rows of x <= 8 NT).  ROWS: weight rows per block (16 or 8).
// GATED: silu(gate) * up epilogue.
// PINGPONG: two rounds of weights in registers, one in use and one on its way (for long k; with a
// single round it would only cost registers, and with them blocks per SM).  The launch bounds keep
// three blocks an SM for up to 8 tokens (two with PINGPONG): a decode step's products have 256 to
// 352 blocks, which should all be resident at once.
// NORM: the epilogue takes part in the norms around the product (`Norm`).
template <int NT, int ROWS, bool GATED, bool PINGPONG, bool NORM, typename OutT>
__global__ void __launch_bounds__(WARPS * 32,
                                  PINGPONG ? (NT <= 2 ? 2 : 1) : (NT <= 2 ? 3 : 1))
linear_small_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                    int ldw, OutT* __restrict__ out, int ldo, int m_rows, int n_out, int k_dim,
                    const Norm norm) {
    constexpr int SETS = GATED ? 2 : 1;              // weight row sets per block
    constexpr bool UPPER = ROWS == 16;               // rows g + 8 of the tile are in use
    __shared__ float red[WARPS][SETS][16][NT * 8 + 1];
    __shared__ float row_factor[NT * 8];

    DE_TRACE_EVENT(n_out, 0);           // (the tag tells the products of a layer apart)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;

    // weight rows of this lane (clamped: rows past the end are computed and dropped)
    const __nv_bfloat16* wrow[SETS][2];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = n0 + g + 8 * h;
            r = r < n_out ? r : n_out - 1;
            wrow[s][h] = w + (size_t)(r + s * n_out) * ldw + 8 * t;
        }
    const __nv_bfloat16* xrow[NT];
    bool xlive[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int m = j * 8 + g;
        xlive[j] = m < m_rows;
        xrow[j] = x + (size_t)(xlive[j] ? m : 0) * ldx + 8 * t;
    }

    float acc[SETS][NT][4];
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[s][j][e] = 0.0f;

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int blocks = (k_dim + KB - 1) / KB;
    // U blocks of k are loaded before any of them is multiplied: enough 16-byte loads in flight
    // per thread (8 to 16) to keep the memory system busy with two or three blocks per SM
    constexpr int U = blocks_per_round(NT, ROWS, GATED);
    typedef uint4 WeightRegs[U][SETS][2][2];
    WeightRegs wa, wb;
    uint4 xv[U][NT][2];

    auto load_weights = [&](WeightRegs& wv, int b0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (b0 + u * WARPS) * KB;
            // a piece past the end of k reads as zero (k is a multiple of 8: pieces are whole)
            const bool ok0 = k0 + 8 * t + 8 <= k_dim, ok1 = k0 + 32 + 8 * t + 8 <= k_dim;
#pragma unroll
            for (int s = 0; s < SETS; ++s)
#pragma unroll
                for (int h = 0; h < (UPPER ? 2 : 1); ++h) {
                    wv[u][s][h][0] = ok0 ? load_stream(wrow[s][h] + k0) : zero;
                    wv[u][s][h][1] = ok1 ? load_stream(wrow[s][h] + k0 + 32) : zero;
                }
        }
    };
    // one round: the tokens' pieces for the round's blocks of k, then the products
    auto multiply = [&](const WeightRegs& wv, int b0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (b0 + u * WARPS) * KB;
            const bool ok0 = k0 + 8 * t + 8 <= k_dim, ok1 = k0 + 32 + 8 * t + 8 <= k_dim;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                xv[u][j][0] = (ok0 && xlive[j]) ? load_cached(xrow[j] + k0) : zero;
                xv[u][j][1] = (ok1 && xlive[j]) ? load_cached(xrow[j] + k0 + 32) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int p = 0; p < 2; ++p)                 // piece
#pragma unroll
                for (int q = 0; q < 2; ++q) {           // half of a piece: one mma step
#pragma unroll
                    for (int s = 0; s < SETS; ++s) {
                        const unsigned a0 = regs(wv[u][s][0][p])[2 * q];
                        const unsigned a2 = regs(wv[u][s][0][p])[2 * q + 1];
                        const unsigned a1 = UPPER ? regs(wv[u][s][1][p])[2 * q] : 0u;
                        const unsigned a3 = UPPER ? regs(wv[u][s][1][p])[2 * q + 1] : 0u;
#pragma unroll
                        for (int j = 0; j < NT; ++j)
                            mma_bf16(acc[s][j], a0, a1, a2, a3, regs(xv[u][j][p])[2 * q],
                                     regs(xv[u][j][p])[2 * q + 1]);
                    }
                }
    };

    load_weights(wa, warp);
    // The next kernel may be launched now: this product's blocks are all resident (one wave), so
    // the next kernel's blocks take nothing from them, and its own first loads (weights, cache
    // rows) overlap this product.  Measured on B200: 2.6% off a decode step against triggering
    // after the main loop.
    pdl_trigger();
    pdl_wait();                                   // x is the previous kernel's output
    DE_TRACE_EVENT(n_out, 1);           // (the tag tells the products of a layer apart)

    // requested now, used in the epilogue: this thread's element of the residual, and the shares
    // of the rows' sums of squares (warp w adds up rows w and w + 8, its lanes every 32nd share)
    float resid_early = 0.0f, sq_sum[NT] = {};
    if constexpr (NORM) {
        if (!GATED && norm.resid != nullptr && threadIdx.x < ROWS * m_rows) {
            const int m = threadIdx.x / ROWS, n = n0 + threadIdx.x % ROWS;
            if (n < n_out) resid_early = norm.resid[(size_t)m * norm.ld_resid + n];
        }
        if (norm.in_parts != nullptr) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int m = warp + 8 * j;
                if (m < m_rows) {
                    const float* parts = norm.in_parts + (size_t)m * norm.in_count;
                    for (int p0 = 0; p0 < norm.in_count; p0 += 256) {      // 8 loads in flight
                        float v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int p = p0 + 32 * i + lane;
                            v[i] = p < norm.in_count ? parts[p] : 0.0f;
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) sq_sum[j] += v[i];
                    }
                }
            }
        }
    }

    // the weights of the next round are requested before this round's are multiplied, so a warp
    // always has a round of loads in flight
    constexpr int ROUND = WARPS * U;
    if constexpr (PINGPONG) {
        for (int b0 = warp; b0 < blocks; b0 += 2 * ROUND) {
            if (b0 + ROUND < blocks) load_weights(wb, b0 + ROUND);
            multiply(wa, b0);
            if (b0 + ROUND >= blocks) break;
            if (b0 + 2 * ROUND < blocks) load_weights(wa, b0 + 2 * ROUND);
            multiply(wb, b0 + ROUND);
        }
    } else {
        for (int b0 = warp; b0 < blocks;) {
            multiply(wa, b0);
            b0 += ROUND;
            if (b0 < blocks) load_weights(wa, b0);
        }
    }

    // add the warps' partial sums
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            red[warp][s][g][j * 8 + 2 * t] = acc[s][j][0];
            red[warp][s][g][j * 8 + 2 * t + 1] = acc[s][j][1];
            red[warp][s][g + 8][j * 8 + 2 * t] = acc[s][j][2];
            red[warp][s][g + 8][j * 8 + 2 * t + 1] = acc[s][j][3];
        }
    if constexpr (NORM) {
        if (norm.in_parts != nullptr) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float total = sq_sum[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                if (lane == 0) row_factor[warp + 8 * j] = rsqrtf(total * norm.inv_width + norm.eps);
            }
        }
    }
    __syncthreads();
    // every thread goes round (the shares of a row's sum of squares are added with shuffles);
    // element e = row m of x, weight row r of the block; the ROWS lanes of a row are neighbours
    for (int e0 = 0; e0 < ROWS * m_rows; e0 += WARPS * 32) {
        const int e = e0 + threadIdx.x;
        const int m = e / ROWS, r = e - m * ROWS;
        const int n = n0 + r;
        const bool live = e < ROWS * m_rows && n < n_out;
        float v[SETS];
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
            float sum = 0.0f;
            if (live) {
#pragma unroll
                for (int wi = 0; wi < WARPS; ++wi) sum += red[wi][s][r][m];
            }
            v[s] = sum;
        }
        if constexpr (NORM) {
            if (norm.in_parts != nullptr && live) {
#pragma unroll
                for (int s = 0; s < SETS; ++s) v[s] *= row_factor[m];
            }
        }
        float y = v[0];
        if constexpr (GATED) {
            // the product's outputs are rounded to bfloat16 before the activation, as a separate
            // product and activation would do
            const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
            const float up = __bfloat162float(__float2bfloat16_rn(v[SETS - 1]));
            y = gate / (1.0f + expf(-gate)) * up;
        }
        if constexpr (NORM && !GATED) {
            if (norm.resid != nullptr) {
                // the branch is rounded to bfloat16 before it joins the residual, as when it goes
                // through memory; the sum and the squares stay float32
                float sum = 0.0f;
                if (live) {
                    const float before = e0 == 0 ? resid_early
                                                 : norm.resid[(size_t)m * norm.ld_resid + n];
                    sum = before + __bfloat162float(__float2bfloat16_rn(y));
                    norm.resid[(size_t)m * norm.ld_resid + n] = sum;
                    y = sum * __bfloat162float(norm.weight[n]);
                }
                float sq = sum * sum;
#pragma unroll
                for (int o = ROWS / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (r == 0 && e < ROWS * m_rows)
                    norm.out_parts[(size_t)m * gridDim.x + blockIdx.x] = sq;
            }
        }
        if (live) out[(size_t)m * ldo + n] = to_out<OutT>(y);
    }
    DE_TRACE_EVENT(n_out, 2);           // (the tag tells the products of a layer apart)
}

template <int NT, int ROWS, bool GATED, bool NORM, typename OutT>
int launch(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int m_rows,
           int n_out, int k_dim, const Norm& norm, cudaStream_t s) {
    const int grid = (n_out + ROWS - 1) / ROWS;
    // more than one round of loads per warp: the gated product has no registers for two rounds
    // with three blocks an SM
    bool rounds = (k_dim + KB - 1) / KB > WARPS * blocks_per_round(NT, ROWS, GATED);
#ifdef LINEAR_SMALL_NO_PINGPONG
    rounds = false;
#endif
    if (rounds && !GATED)
        return de_launch(linear_small_kernel<NT, ROWS, GATED, true, NORM, OutT>, dim3(grid),
                         dim3(WARPS * 32), 0, s, (const __nv_bfloat16*)x, ldx,
                         (const __nv_bfloat16*)w, ldw, (OutT*)out, ldo, m_rows, n_out, k_dim, norm);
    return de_launch(linear_small_kernel<NT, ROWS, GATED, false, NORM, OutT>, dim3(grid),
                     dim3(WARPS * 32), 0, s, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w,
                     ldw, (OutT*)out, ldo, m_rows, n_out, k_dim, norm);
}

// few weight rows: blocks of 8 rows, so that there are blocks for every SM
#ifndef FEW_ROWS_LIMIT
#define FEW_ROWS_LIMIT (16 * 2 * 148)
#endif
bool few_rows(int n_out) { return n_out < FEW_ROWS_LIMIT; }

template <bool GATED, bool NORM, typename OutT>
int pick(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int m_rows,
         int n_out, int k_dim, const Norm& norm, cudaStream_t s) {
#define GO(NT)                                                                                   \
    return few_rows(n_out) ? launch<NT, 8, GATED, NORM, OutT>(x, ldx, w, ldw, out, ldo, m_rows,  \
                                                               n_out, k_dim, norm, s)            \
                           : launch<NT, 16, GATED, NORM, OutT>(x, ldx, w, ldw, out, ldo, m_rows, \
                                                                n_out, k_dim, norm, s)
    if (m_rows <= 8) { GO(1); }
    if (m_rows <= 16) { GO(2); }
    if constexpr (NORM) return -5; else { GO(4); }
#undef GO
}

int check(int m_rows, int k_dim, int ldx, int ldw, const void* x, const void* w) {
    if (m_rows > 32 || k_dim <= 0) return -2;
    // 16-byte pieces: k a multiple of 8, rows that start on 16-byte boundaries
    if (k_dim % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return -3;
    return 0;
}

}  // namespace

DE_EXPORT int de_linear_small_max_rows() { return 32; }

// out_f32: 1 for float32 output, 0 for bfloat16.  gated: w is [2 * n_out, k], gate rows first.
DE_EXPORT int de_linear_small(const void* x, int ldx, const void* w, int ldw, void* out, int ldo,
                              int m_rows, int n_out, int k_dim, int out_f32, int gated,
                              void* stream) {
    if (m_rows <= 0 || n_out <= 0) return 0;
    if (int code = check(m_rows, k_dim, ldx, ldw, x, w)) return code;
    cudaStream_t s = (cudaStream_t)stream;
    const Norm none = {};
    if (gated) {
        if (out_f32) return -4;
        return pick<true, false, __nv_bfloat16>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim,
                                                none, s);
    }
    if (out_f32)
        return pick<false, false, float>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim, none, s);
    return pick<false, false, __nv_bfloat16>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim, none, s);
}

// How many shares of a row's sum of squares a product with n_out outputs leaves (its blocks).
DE_EXPORT int de_linear_small_parts(int n_out) {
    return (n_out + (few_rows(n_out) ? 8 : 16) - 1) / (few_rows(n_out) ? 8 : 16);
}

// The same product (bfloat16 output, up to 16 rows) taking part in the norms around it.
// in_parts [m_rows, in_count] (or null): x lacks the factor of the norm before the product, which
// follows from these shares of the rows' sums of squares over `width` elements.
// resid [m_rows, ld_resid] float32 (or null): the result joins the residual, out becomes residual *
// norm_weight, and out_parts [m_rows, de_linear_small_parts(n_out)] receives the new shares.
DE_EXPORT int de_linear_small_norm(const void* x, int ldx, const void* w, int ldw, void* out,
                                   int ldo, int m_rows, int n_out, int k_dim, int gated,
                                   const float* in_parts, int in_count, int width, float eps,
                                   float* resid, int ld_resid, const void* norm_weight,
                                   float* out_parts, void* stream) {
    if (m_rows <= 0 || n_out <= 0) return 0;
    if (int code = check(m_rows, k_dim, ldx, ldw, x, w)) return code;
    if (m_rows > 16) return -5;
    if (in_parts != nullptr && (in_count <= 0 || width <= 0)) return -6;
    if (resid != nullptr && (norm_weight == nullptr || out_parts == nullptr || gated)) return -6;
    Norm norm = {};
    norm.in_parts = in_parts;
    norm.in_count = in_count;
    norm.inv_width = width > 0 ? 1.0f / (float)width : 0.0f;
    norm.eps = eps;
    norm.resid = resid;
    norm.ld_resid = ld_resid;
    norm.weight = (const __nv_bfloat16*)norm_weight;
    norm.out_parts = out_parts;
    cudaStream_t s = (cudaStream_t)stream;
    if (gated)
        return pick<true, true, __nv_bfloat16>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim,
                                               norm, s);
    return pick<false, true, __nv_bfloat16>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim, norm, s);
}

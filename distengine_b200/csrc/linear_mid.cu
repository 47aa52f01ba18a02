// Matrix products for 17 to 128 tokens (decode steps of many requests, short prompt portions):
// out[t, n] = sum_k x[t, k] * w[n, k], bfloat16 operands, float32 accumulation, on the
// 5th-generation tensor cores.  Such a product still only streams the weights once, so the roles of
// the operands are swapped against a prompt's product: the 128 lanes of tensor memory are 128 rows
// of w (the M side of tcgen05.mma) and the tokens are the N side (padded to a multiple of 16), so
// that no tensor-core work is spent on rows that do not exist.
//
// Work: one block per (128 rows of w, slice of k).  The slices of a tile's k are the blocks of a
// thread-block cluster (1, 2, 4 or 8); each keeps its partial sums [tokens][128] in its own shared
// memory, and after a cluster barrier every block adds up, through distributed shared memory, the
// partial sums of its share of the tokens and writes them (so the sum over k is made in a fixed
// order and nothing goes through global memory).  The host picks the split so that all SMs pull
// weights.
//
// A block needs about 100 KB of shared memory, half an SM's, and at most 256 columns of tensor
// memory: the blocks of the next product fit beside those of the running one, and because the
// weights are no kernel's output a block requests its first tiles of w before it waits for the
// kernel before it (programmatic dependent launch) - the weight stream does not stop at a kernel's
// end.
//
// Roles: warp 0, one thread: TMA loads (128 x 64 tiles of w, tokens x 64 tiles of x, 128-byte
// swizzle, zero fill outside the matrices); warp 1, one thread: tcgen05.mma, M = 128, N = tokens;
// warps 2-5: the rows' factors of a norm before the product, then the accumulator out of tensor
// memory.  Epilogues, in the adding-up phase: silu(gate) * up when w stacks gate rows over up rows
// (a block then holds 128 gate rows and the 128 up rows that belong to them, two accumulators;
// src/layers/activation.py:6-9, src/models/llama.py:23-27), and the norms around the product as in
// linear_small.cu (`Norm`).  Every wait on an mbarrier is bounded (status 3).
//
// Stands where the reference calls F.linear (src/layers/linear.py:19-20).

#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_common.cuh"
#include "tensor_maps.cuh"

DE_DEFINE_PDL_SWITCH

namespace cg = cooperative_groups;
using namespace tc5;

namespace {

constexpr int BM = 128;                // rows of w per block = lanes of tensor memory
constexpr int BK = 64;                 // k per stage: 128 bytes of bfloat16 = one swizzle row
constexpr int THREADS = 192;           // producer warp, tensor-core warp, four epilogue warps
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int MAX_TOKENS = 128;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_BUDGET = 100 * 1024;   // tiles of a block: two blocks an SM
constexpr int MAX_SPLIT = 8;

// What the epilogue does for the norms around a product (all pointers may be null); as in
// linear_small.cu, with one share of a row's sum of squares per 128 outputs.
struct Norm {
    const float* in_parts;             // [tokens][in_count]
    int in_count;
    float inv_width, eps;
    float* resid;                      // [tokens][ld_resid] float32, takes the sum
    int ld_resid;
    const __nv_bfloat16* weight;       // [n_out]
    float* out_parts;                  // [tokens][gridDim.y]
};

__host__ __device__ constexpr int round_up(int v, int to) { return (v + to - 1) / to * to; }

#ifdef LINEAR_MID_TIMING
// Debugging aid, compiled on request only: wall-clock stamps of one block's phases.
__device__ unsigned long long mid_stamps[16];
#define STAMP(k)                                                                       \
    do {                                                                               \
        if (blockIdx.y == LINEAR_MID_TIMING && blockIdx.x == 0 && stamp_on) {          \
            unsigned long long t_;                                                     \
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t_));                   \
            mid_stamps[k] = t_;                                                        \
        }                                                                              \
    } while (0)
#else
#define STAMP(k) do { } while (0)
#endif

// bytes of a stage: the tile(s) of w, then the tile of x (tokens x 64), 1024-byte aligned
__host__ __device__ constexpr int stage_bytes(bool gated, int n_pad) {
    return (gated ? 2 : 1) * A_BYTES + round_up(n_pad * BK * 2, 1024);
}
__host__ __device__ constexpr int partial_bytes(bool gated, int n_pad) {
    return (gated ? 2 : 1) * n_pad * BM * 4;
}
__host__ __device__ inline int stage_count(bool gated, int n_pad) {
    int stages = SMEM_BUDGET / stage_bytes(gated, n_pad);
    stages = stages < 2 ? 2 : (stages > MAX_STAGES ? MAX_STAGES : stages);
    // the partial sums take the tiles' place afterwards
    while (stages * stage_bytes(gated, n_pad) < partial_bytes(gated, n_pad)) ++stages;
    return stages;
}

template <bool GATED>
__global__ void __launch_bounds__(THREADS, 2)
linear_mid_kernel(const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_up,
                  const __grid_constant__ CUtensorMap map_x, void* __restrict__ out_raw, int ldo,
                  int out_f32, int tokens, int n_out, int k_dim, int n_pad, int stages,
                  const Norm norm, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
    __shared__ __align__(8) unsigned long long acc_done;
    __shared__ unsigned tmem_base_slot;
    __shared__ float factor_s[MAX_TOKENS];          // the rows' factors of the norm before

#ifdef LINEAR_MID_TIMING
#ifndef LINEAR_MID_TIMING_N
#define LINEAR_MID_TIMING_N 0
#define LINEAR_MID_TIMING_K 0
#endif
    const bool stamp_on = LINEAR_MID_TIMING_N == 0 ||
                          (n_out == LINEAR_MID_TIMING_N && k_dim == LINEAR_MID_TIMING_K);
#endif
    if (threadIdx.x == 0) STAMP(0);
    cg::cluster_group cluster = cg::this_cluster();
    const int split = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.y, n0 = tile * BM;
    const int k_steps_all = (k_dim + BK - 1) / BK;
    const int ks_begin = (int)((long long)k_steps_all * rank / split);
    const int ks_end = (int)((long long)k_steps_all * (rank + 1) / split);
    const int k_steps = ks_end - ks_begin;
    const int a_bytes = (GATED ? 2 : 1) * A_BYTES;
    const int b_bytes = n_pad * BK * 2;
    const int stride = stage_bytes(GATED, n_pad);
    const unsigned tmem_cols = (GATED ? 2u : 1u) * (n_pad <= 32 ? 32u : (n_pad <= 64 ? 64u : 128u));

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, tmem_cols);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;
    if (threadIdx.x == 0) STAMP(1);
    // the next kernel may be launched: its blocks fit beside these and start on their own weights
    pdl_trigger();

    bool ok = true;
    if (warp == 0) {
        // ---- producer.  The weights of the first stages are requested before the wait for the
        // kernel before this one; x, its output, after it.
        if (lane == 0) {
            const int early = k_steps < stages ? k_steps : stages;
            for (int it = 0; it < early; ++it) {
                unsigned char* a_tile = tiles + it * stride;
                mbar_expect_tx(&full_bar[it], a_bytes + b_bytes);
                tma_load_2d(a_tile, &map_w, &full_bar[it], (ks_begin + it) * BK, n0);
                if (GATED)
                    tma_load_2d(a_tile + A_BYTES, &map_up, &full_bar[it], (ks_begin + it) * BK, n0);
            }
            STAMP(2);
            pdl_wait();
            STAMP(3);
            for (int it = 0; it < early; ++it)
                tma_load_2d(tiles + it * stride + a_bytes, &map_x, &full_bar[it],
                            (ks_begin + it) * BK, 0);
            STAMP(4);
            for (int it = early; it < k_steps && ok; ++it) {
                const int s = it % stages;
                ok = mbar_wait(&empty_bar[s], ((it / stages) - 1) & 1, status);
                if (!ok) break;
                unsigned char* a_tile = tiles + s * stride;
                mbar_expect_tx(&full_bar[s], a_bytes + b_bytes);
                tma_load_2d(a_tile, &map_w, &full_bar[s], (ks_begin + it) * BK, n0);
                if (GATED)
                    tma_load_2d(a_tile + A_BYTES, &map_up, &full_bar[s], (ks_begin + it) * BK, n0);
                tma_load_2d(a_tile + a_bytes, &map_x, &full_bar[s], (ks_begin + it) * BK, 0);
            }
        }
    } else if (warp == 1) {
        // ---- tensor core
        if (lane == 0) {
            const unsigned idesc = instr_desc(BM, n_pad);
            const unsigned up_cols = tmem_cols / 2;          // GATED: the up accumulator's columns
            for (int it = 0; it < k_steps && ok; ++it) {
                const int s = it % stages;
                ok = mbar_wait(&full_bar[s], (it / stages) & 1, status);
                if (!ok) break;
                if (it == 0) STAMP(5);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* a_tile = tiles + s * stride;
                const unsigned long long a_desc = smem_desc(a_tile);
                const unsigned long long b_desc = smem_desc(a_tile + a_bytes);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, it > 0 || k > 0);
                    if (GATED)
                        umma_bf16(tmem_base + up_cols, smem_desc(a_tile + A_BYTES) + 2 * k,
                                  b_desc + 2 * k, idesc, it > 0 || k > 0);
                }
                umma_commit(&empty_bar[s]);
            }
            umma_commit(&acc_done);
            STAMP(6);
        }
    } else {
        // ---- epilogue warps.  While the product runs: the factors of the norm before it, for
        // the tokens this block adds up (warp q takes every fourth of them).
        pdl_wait();
        const int q = warp & 3;
        const int per_block = (tokens + split - 1) / split;
        const int t_begin = rank * per_block;
        const int t_end = min(tokens, t_begin + per_block);
        if (norm.in_parts != nullptr) {
            for (int t = t_begin + q; t < t_end; t += 4) {
                const float* parts = norm.in_parts + (size_t)t * norm.in_count;
                float sum = 0.0f;
                for (int p0 = 0; p0 < norm.in_count; p0 += 128) {
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int p = p0 + 32 * i + lane;
                        v[i] = p < norm.in_count ? parts[p] : 0.0f;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) sum += v[i];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (lane == 0) factor_s[t - t_begin] = rsqrtf(sum * norm.inv_width + norm.eps);
            }
        }
        // the accumulator: thread = row of w; partial[half][token][row]
        if (k_steps > 0) ok = mbar_wait(&acc_done, 0, status);
        if (threadIdx.x == 64) STAMP(7);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        float* partial = reinterpret_cast<float*>(tiles);
        const int row = q * 32 + lane;
        const unsigned lane_base = tmem_base + ((unsigned)(q * 32) << 16);
#pragma unroll 1
        for (int half = 0; half < (GATED ? 2 : 1); ++half) {
#pragma unroll 1
            for (int c = 0; c < n_pad; c += 32) {
                unsigned v[32];
                if (k_steps > 0 && ok) {
                    tmem_load_32cols(lane_base + half * (tmem_cols / 2) + c, v);
                    tmem_wait_loads();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;       // a slice without any k
                }
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (c + i < n_pad)
                        partial[(size_t)(half * n_pad + c + i) * BM + row] = __uint_as_float(v[i]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        if (threadIdx.x == 64) STAMP(8);
    }

    // ---- the sum over the slices of k: block `rank` adds up its share of the tokens.  A warp
    // takes a token, a lane four neighbouring rows of w (16-byte loads from the blocks' shared
    // memory, 8-byte stores), so a token's sum of squares is one warp's.
    cluster.sync();
    if (threadIdx.x == 64) STAMP(9);
    if (warp >= 2) {
        constexpr int HALVES = GATED ? 2 : 1;
        const int n = n0 + 4 * lane;
        const int per_block = (tokens + split - 1) / split;
        const int t_begin = rank * per_block;
        const int t_end = min(tokens, t_begin + per_block);
        const float* partial = reinterpret_cast<const float*>(tiles);
        const float* remote[MAX_SPLIT];
#pragma unroll
        for (int c = 0; c < MAX_SPLIT; ++c)
            remote[c] = c < split ? cluster.map_shared_rank(partial, c) : partial;
        float w_norm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (!GATED && norm.resid != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (n + e < n_out) w_norm[e] = __bfloat162float(norm.weight[n + e]);
        }
        // all four rows exist, and rows of out and of the residual start on 16-byte boundaries
        const bool whole = n + 3 < n_out && ldo % 4 == 0 &&
                           (reinterpret_cast<uintptr_t>(out_raw) & 15) == 0 &&
                           (norm.resid == nullptr ||
                            (norm.ld_resid % 4 == 0 &&
                             (reinterpret_cast<uintptr_t>(norm.resid) & 15) == 0));
        // TB tokens a round: everything they need is requested before any of it is used
        constexpr int TB = 1;
        for (int t0 = t_begin + (warp - 2); t0 < t_end; t0 += 4 * TB) {
            float4 part[TB][HALVES][MAX_SPLIT];
            float before[TB][4];
#pragma unroll
            for (int i = 0; i < TB; ++i) {
                const int t = min(t0 + 4 * i, t_end - 1);
#pragma unroll
                for (int half = 0; half < HALVES; ++half)
#pragma unroll
                    for (int c = 0; c < MAX_SPLIT; ++c)
                        part[i][half][c] = c < split
                            ? *reinterpret_cast<const float4*>(
                                  remote[c] + (size_t)(half * n_pad + t) * BM + 4 * lane)
                            : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int e = 0; e < 4; ++e) before[i][e] = 0.0f;
                if (!GATED && norm.resid != nullptr) {
                    const float* r = norm.resid + (size_t)t * norm.ld_resid + n;
                    if (whole) {
                        const float4 b4 = *reinterpret_cast<const float4*>(r);
                        before[i][0] = b4.x; before[i][1] = b4.y;
                        before[i][2] = b4.z; before[i][3] = b4.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < n_out) before[i][e] = r[e];
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < TB; ++i) {
                const int t = t0 + 4 * i;
                if (t >= t_end) break;                         // uniform over the warp
                float v[HALVES][4];
#pragma unroll
                for (int half = 0; half < HALVES; ++half) {
                    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int c = 0; c < MAX_SPLIT; ++c) {
                        sum.x += part[i][half][c].x; sum.y += part[i][half][c].y;
                        sum.z += part[i][half][c].z; sum.w += part[i][half][c].w;
                    }
                    const float f = norm.in_parts != nullptr ? factor_s[t - t_begin] : 1.0f;
                    v[half][0] = sum.x * f; v[half][1] = sum.y * f;
                    v[half][2] = sum.z * f; v[half][3] = sum.w * f;
                }
                float y[4], sq = 0.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    y[e] = v[0][e];
                    if (GATED) {
                        // the product's outputs are rounded to bfloat16 before the activation,
                        // as a separate product and activation would do
                        const float gate = __bfloat162float(__float2bfloat16_rn(v[0][e]));
                        const float up = __bfloat162float(__float2bfloat16_rn(v[HALVES - 1][e]));
                        y[e] = gate / (1.0f + expf(-gate)) * up;
                    }
                    if (!GATED && norm.resid != nullptr) {
                        // the branch is rounded to bfloat16 before it joins the residual, as when
                        // it goes through memory; the sum and the squares stay float32
                        const float sum =
                            n + e < n_out
                                ? before[i][e] + __bfloat162float(__float2bfloat16_rn(y[e]))
                                : 0.0f;
                        before[i][e] = sum;
                        y[e] = sum * w_norm[e];
                        sq += sum * sum;
                    }
                }
                if (!GATED && norm.resid != nullptr) {
                    float* r = norm.resid + (size_t)t * norm.ld_resid + n;
                    if (whole) {
                        *reinterpret_cast<float4*>(r) =
                            make_float4(before[i][0], before[i][1], before[i][2], before[i][3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < n_out) r[e] = before[i][e];
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    if (lane == 0) norm.out_parts[(size_t)t * gridDim.y + tile] = sq;
                }
                if (out_f32) {
                    float* o = reinterpret_cast<float*>(out_raw) + (size_t)t * ldo + n;
                    if (whole) {
                        *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < n_out) o[e] = y[e];
                    }
                } else {
                    __nv_bfloat16* o =
                        reinterpret_cast<__nv_bfloat16*>(out_raw) + (size_t)t * ldo + n;
                    if (whole) {
                        *reinterpret_cast<uint2*>(o) =
                            make_uint2(pack2(y[0], y[1]), pack2(y[2], y[3]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (n + e < n_out) o[e] = __float2bfloat16_rn(y[e]);
                    }
                }
            }
        }
    }
    if (threadIdx.x == 64) STAMP(10);
    cluster.sync();                    // nobody leaves while its shared memory may still be read
    if (threadIdx.x == 64) STAMP(11);
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

int pick_split(int tiles, int k_steps, int sms) {
    // as many slices of k as keep every block's place among two blocks an SM, and no slice empty
    int split = 1;
#ifndef LINEAR_MID_BLOCKS_PER_SM
#define LINEAR_MID_BLOCKS_PER_SM 2
#endif
#ifndef LINEAR_MID_MAX_SPLIT
#define LINEAR_MID_MAX_SPLIT MAX_SPLIT
#endif
    while (split * 2 <= LINEAR_MID_MAX_SPLIT && tiles * split * 2 <= LINEAR_MID_BLOCKS_PER_SM * sms &&
           split * 2 <= k_steps)
        split *= 2;
    return split;
}

template <bool GATED>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_up, const CUtensorMap& map_x, void* out,
           int ldo, int out_f32, int tokens, int n_out, int k_dim, const Norm& norm, int split,
           int* status, cudaStream_t stream) {
    const int n_pad = round_up(tokens, 16);
    const int stages = stage_count(GATED, n_pad);
    const size_t smem = (size_t)stages * stage_bytes(GATED, n_pad) + 1024;
    static bool sized = false;
    if (!sized) {
        cudaError_t e = cudaFuncSetAttribute(linear_mid_kernel<GATED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        sized = true;
    }
    de_prefer_carveout(linear_mid_kernel<GATED>, 100);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)split, (unsigned)((n_out + BM - 1) / BM));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 2 : 1;
    return de_check(cudaLaunchKernelEx(&cfg, linear_mid_kernel<GATED>, map_w, map_up, map_x, out, ldo,
                                       out_f32, tokens, n_out, k_dim, n_pad, stages, norm, status));
}

}  // namespace

#ifdef LINEAR_MID_TIMING
DE_EXPORT int de_linear_mid_stamps(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, mid_stamps, sizeof(mid_stamps));
}
#endif
DE_EXPORT int de_linear_mid_max_rows() { return MAX_TOKENS; }
// How many shares of a row's sum of squares a product with n_out outputs leaves (its row tiles).
DE_EXPORT int de_linear_mid_parts(int n_out) { return (n_out + BM - 1) / BM; }

// x [tokens, k] and w [n_out, k] (gated: [2 n_out, k], gate rows first) bfloat16 with contiguous
// rows, out [tokens, n_out] bfloat16 or float32 (out_f32).  The norm arguments as in
// de_linear_small_norm: in_parts [tokens, in_count] or null; resid [tokens, ld_resid], norm_weight
// [n_out] and out_parts [tokens, de_linear_mid_parts(n_out)] or null.  `split` 0: chosen here.
// `status` receives 3 if a wait inside the kernel ran out.
DE_EXPORT int de_linear_mid(const void* x, int ldx, const void* w, int ldw, void* out, int ldo,
                            int tokens, int n_out, int k_dim, int out_f32, int gated,
                            const float* in_parts, int in_count, int width, float eps,
                            float* resid, int ld_resid, const void* norm_weight, float* out_parts,
                            int split, int* status, void* stream) {
    if (tokens <= 0 || n_out <= 0) return 0;
    if (tokens > MAX_TOKENS || k_dim <= 0) return -2;
    if (k_dim % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return -3;
    if (gated && out_f32) return -4;
    if (in_parts != nullptr && (in_count <= 0 || width <= 0)) return -6;
    if (resid != nullptr && (norm_weight == nullptr || out_parts == nullptr || gated || out_f32))
        return -6;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    const int tiles = (n_out + BM - 1) / BM, k_steps = (k_dim + BK - 1) / BK;
    if (split <= 0) split = pick_split(tiles, k_steps, sms);
    if (split > MAX_SPLIT || (split & (split - 1))) return -4;
    Norm norm = {};
    norm.in_parts = in_parts;
    norm.in_count = in_count;
    norm.inv_width = width > 0 ? 1.0f / (float)width : 0.0f;
    norm.eps = eps;
    norm.resid = resid;
    norm.ld_resid = ld_resid;
    norm.weight = (const __nv_bfloat16*)norm_weight;
    norm.out_parts = out_parts;
    const int n_pad = round_up(tokens, 16);
    CUtensorMap map_w, map_up, map_x;
    int code = tensor_maps::get(&map_x, x, tokens, k_dim, ldx, n_pad, BK);
    if (code) return code;
    code = tensor_maps::get(&map_w, w, n_out, k_dim, ldw, BM, BK);
    if (code) return code;
    map_up = map_w;
    if (gated) {
        code = tensor_maps::get(&map_up, (const __nv_bfloat16*)w + (size_t)n_out * ldw, n_out, k_dim,
                                ldw, BM, BK);
        if (code) return code;
        return launch<true>(map_w, map_up, map_x, out, ldo, 0, tokens, n_out, k_dim, norm, split,
                            status, (cudaStream_t)stream);
    }
    return launch<false>(map_w, map_up, map_x, out, ldo, out_f32, tokens, n_out, k_dim, norm, split,
                         status, (cudaStream_t)stream);
}

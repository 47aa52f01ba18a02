// bfloat16 matrix product on the 5th-generation tensor cores: out[m, n] = sum_k x[m, k] * w[n, k],
// float32 accumulation in tensor memory, for prompt portions (many rows of x).
//
// A persistent kernel, one block per SM, each block walking over 128 x bn tiles of the output
// (bn a multiple of 32 up to 256, chosen by the host so that the last round of tiles over the SMs
// wastes least), with the roles split over warps:
//   * warp 0, one thread: moves 128 x 64 tiles of x and bn x 64 tiles of w into shared memory with
//     TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill outside the matrices), 4 stages
//     deep, each stage guarded by a "full" mbarrier with a transaction count;
//   * warp 1, one thread: issues tcgen05.mma (kind::f16, M = 128, N = bn, K = 16; operands are
//     shared-memory descriptors), four per stage, hands the stage back with tcgen05.commit on its
//     "empty" mbarrier, and after a tile's last stage commits on the accumulator's "full" mbarrier;
//   * warps 2-5: the epilogue.  The accumulator is double-buffered in tensor memory (2 x 256
//     columns), so these warps read one tile with tcgen05.ld, convert and store it while the
//     tensor core already works on the next.  The gated epilogue computes silu(gate) * up from the
//     two halves of the accumulator (src/layers/activation.py:6-9), so the activation costs no
//     pass over memory and the product's [gate | up] output is never written.
// Tiles are numbered with the rows of x fastest, so the blocks at work share a few tiles of w.
// No cluster launch; every block fetches its own tiles.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls a thread records status 3, stops
// waiting, and the block runs to its end (tensor memory is freed on every path); the host raises.
//
// Stands where the reference calls F.linear (src/layers/linear.py:19-20) on [1, T, H] inputs.

#include <cuda.h>

#include "common.cuh"
#include "tcgen05_common.cuh"
#include "tensor_maps.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int BM = 128;                // rows of x per tile = lanes of tensor memory
constexpr int BK = 64;                 // k per stage: 128 bytes of bfloat16 = one swizzle row
constexpr int THREADS = 192;           // producer warp, tensor-core warp, four epilogue warps
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int MAX_BN = 256;            // columns of an accumulator
constexpr int STAGES = 4;
constexpr int STAGE_BYTES = A_BYTES + MAX_BN * BK * 2;   // 48 KB: room for the widest tile of w
constexpr int SMEM_TILES = STAGES * STAGE_BYTES;

using namespace tc5;

// One tile's accumulator out of tensor memory: thread = row.  GATED: columns 0 .. bn/2-1 are gate
// outputs, bn/2 .. bn-1 the up outputs of the same features; bn/2 columns of silu(gate) * up go out.
template <bool GATED, typename OutT>
__device__ __forceinline__ void store_tile(unsigned lane_base, int bn, OutT* out_row, bool row_live,
                                           int cols_left, bool vec) {
    if (GATED) {
#pragma unroll 1
        for (int c = 0; c < bn / 2; c += 32) {
            unsigned gate[32], up[32];
            tmem_load_32cols(lane_base + c, gate);
            tmem_load_32cols(lane_base + bn / 2 + c, up);
            tmem_wait_loads();
            if (!row_live) continue;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                float y[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // product outputs are rounded to bfloat16 before the activation, as a
                    // separate product and activation kernel would do
                    const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gate[i + j])));
                    const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(up[i + j])));
                    // fast division: a gate far below zero gives 0, the function's limit
                    y[j] = __fdividef(g, 1.0f + __expf(-g)) * u;
                }
                if (vec && c + i + 8 <= cols_left) {
                    store8(out_row + c + i, y);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (c + i + j < cols_left) out_row[c + i + j] = from_float<OutT>(y[j]);
                }
            }
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < bn; c += 32) {
            unsigned v[32];
            tmem_load_32cols(lane_base + c, v);
            tmem_wait_loads();
            if (!row_live) continue;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                float y[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = __uint_as_float(v[i + j]);
                const int col = c + i;
                if (vec && col + 8 <= cols_left) {
                    store8(out_row + col, y);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (col + j < cols_left) out_row[col + j] = from_float<OutT>(y[j]);
                }
            }
        }
    }
}

// map_w: the rows of w (GATED: the gate rows); map_up: the up rows (GATED only).
template <bool GATED, typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_up, OutT* __restrict__ out, int ldo,
                    int m_rows, int n_out, int k_dim, int bn, int tiles_m, int tiles_n,
                    int* status) {
    const int b_bytes = bn * BK * 2;
    const int out_cols = GATED ? bn / 2 : bn;             // output columns of a tile
    constexpr unsigned TMEM_COLS = 2 * MAX_BN;            // two accumulators
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the tiles need 1024-byte alignment for the swizzle pattern
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_steps = (k_dim + BK - 1) / BK;
    const int total = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);                  // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;

    bool ok = true;
    if (warp == 0) {
        // ---- producer: TMA loads, ahead of the tensor core by up to STAGES
        pdl_wait();                                        // x is the previous kernel's output
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
                for (int ks = 0; ks < k_steps; ++ks, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES) ok = mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1, status);
                    if (!ok) break;
                    unsigned char* a_tile = tiles + s * STAGE_BYTES;
                    unsigned char* b_tile = a_tile + A_BYTES;
                    mbar_expect_tx(&full_bar[s], A_BYTES + b_bytes);
                    tma_load_2d(a_tile, &map_x, &full_bar[s], ks * BK, tile_m * BM);
                    if (GATED) {
                        tma_load_2d(b_tile, &map_w, &full_bar[s], ks * BK, tile_n * (bn / 2));
                        tma_load_2d(b_tile + b_bytes / 2, &map_up, &full_bar[s], ks * BK,
                                    tile_n * (bn / 2));
                    } else {
                        tma_load_2d(b_tile, &map_w, &full_bar[s], ks * BK, tile_n * bn);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor core: four K = 16 steps per stage, accumulators in tensor memory
        if (lane == 0) {
            const unsigned idesc = instr_desc(BM, bn);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                // the epilogue has read this accumulator's tile before last
                if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, status);
                for (int ks = 0; ks < k_steps && ok; ++ks, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, status);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* a_tile = tiles + s * STAGE_BYTES;
                    const unsigned long long a_desc = smem_desc(a_tile);
                    const unsigned long long b_desc = smem_desc(a_tile + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 elements of k are 32 bytes: the start addresses advance by 2
                        umma_bf16(tmem_base + buf * MAX_BN, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                  ks > 0 || k > 0);
                    }
                    umma_commit(&empty_bar[s]);            // the stage is free when these are done
                }
                umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ---- epilogue: warp w reads the lanes 32 (w % 4) .. + 31 of the accumulator
        const int quarter = warp & 3;
        const bool vec = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
        int local = 0;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++local) {
            const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
            const int buf = local & 1;
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, status);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int row = tile_m * BM + quarter * 32 + lane;
            const unsigned lane_base = tmem_base + buf * MAX_BN + ((unsigned)(quarter * 32) << 16);
            OutT* out_row = out + (size_t)row * ldo + (size_t)tile_n * out_cols;
            store_tile<GATED, OutT>(lane_base, bn, out_row, row < m_rows,
                                    n_out - tile_n * out_cols, vec);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    __syncwarp();
    pdl_trigger();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------- host side
// A [rows, k] bfloat16 matrix with row stride ld (elements), boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    return tensor_maps::get(map, base, rows, k, ld, box_rows, BK);
}

int sm_count() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            count <= 0)
            count = 148;
    }
    return count;
}

// The tile width: the candidate whose rounds of tiles over the SMs take least, a round of tiles
// bn wide taking about bn + 16 units.  Tiles narrower than 128 read too much of x and w per flop;
// they are candidates only when wider ones would leave SMs without a tile.
int choose_bn(int m_rows, int n_out, bool gated) {
    const int tiles_m = (m_rows + BM - 1) / BM;
    const long sms = sm_count();
    auto tiles = [&](int bn) {
        const int cols = gated ? bn / 2 : bn;
        return (long)tiles_m * ((n_out + cols - 1) / cols);
    };
    int best = 0;
    long best_cost = 0;
    const bool small = tiles(128) < sms;
    const int step = gated ? 64 : 32;
    for (int bn = MAX_BN; bn >= (small ? step : 128); bn -= step) {
        const long cost = ((tiles(bn) + sms - 1) / sms) * (bn + 16);
        if (best == 0 || cost < best_cost) {
            best = bn;
            best_cost = cost;
        }
    }
    return best;
}

template <bool GATED, typename OutT>
int launch(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int m_rows, int n_out,
           int k_dim, int* status, cudaStream_t s) {
    const int bn = choose_bn(m_rows, n_out, GATED);
    CUtensorMap map_x, map_w, map_up;
    int code = make_map(&map_x, x, m_rows, k_dim, ldx, BM);
    if (code) return code;
    // gated: the gate rows and the up rows as matrices of their own, so that a tile at the edge
    // reads zeros and not the other's rows
    code = make_map(&map_w, w, n_out, k_dim, ldw, GATED ? bn / 2 : bn);
    if (code) return code;
    const void* up = GATED ? (const void*)((const __nv_bfloat16*)w + (size_t)n_out * ldw) : w;
    code = make_map(&map_up, up, n_out, k_dim, ldw, GATED ? bn / 2 : bn);
    if (code) return code;
    const size_t smem = (size_t)SMEM_TILES + 1024;
    auto kernel = gemm_tcgen05_kernel<GATED, OutT>;
    static bool sized = false;                 // per instantiation: the attribute is set once
    if (!sized) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        sized = true;
    }
    const int out_cols = GATED ? bn / 2 : bn;
    const int tiles_m = (m_rows + BM - 1) / BM, tiles_n = (n_out + out_cols - 1) / out_cols;
    const int total = tiles_m * tiles_n;
    const int grid = total < sm_count() ? total : sm_count();
    return de_launch(kernel, dim3(grid), dim3(THREADS), smem, s, map_x, map_w, map_up, (OutT*)out,
                     ldo, m_rows, n_out, k_dim, bn, tiles_m, tiles_n, status);
}

}  // namespace

// The tile width the kernel would take for this shape (the host decides with it whether the
// shape suits the kernel).
DE_EXPORT int de_gemm_tcgen05_tile(int m_rows, int n_out, int gated) {
    return choose_bn(m_rows, n_out, gated != 0);
}
DE_EXPORT int de_gemm_tcgen05_sms() { return sm_count(); }

// out_f32: float32 output (not with gated).  gated: w is [2 n_out, k] with the gate rows first; out
// is [m, n_out] = silu(x gate^T) * (x up^T).  x, w: bfloat16, rows contiguous, 16-byte aligned
// row starts.  `status` receives 3 if a wait inside the kernel ran out.
DE_EXPORT int de_gemm_tcgen05(const void* x, int ldx, const void* w, int ldw, void* out, int ldo,
                              int m_rows, int n_out, int k_dim, int out_f32, int gated, int* status,
                              void* stream) {
    if (m_rows <= 0 || n_out <= 0) return 0;
    if (k_dim <= 0 || k_dim % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)x & 15) ||
        ((uintptr_t)w & 15))
        return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (gated) {
        if (out_f32) return -5;
        return launch<true, __nv_bfloat16>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim, status, s);
    }
    if (out_f32)
        return launch<false, float>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim, status, s);
    return launch<false, __nv_bfloat16>(x, ldx, w, ldw, out, ldo, m_rows, n_out, k_dim, status, s);
}

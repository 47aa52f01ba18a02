// One persistent kernel for a whole decode step of a pre-norm decoder (RMS norm, grouped-query
// attention with rotary position encoding over the paged cache, gated feed-forward): embedding,
// every layer, final norm and output matrix in a single cooperative launch, one block per SM,
// phases separated by grid-wide barriers.  For up to 16 tokens (each the next token of its own
// request), bfloat16 weights and cache.  Compiled per head size (-DHEAD_DIM=d, d a multiple of 32).
//
// Why: at this size a step is a stream of weights (every matrix is read once) and of ~200 tiny
// dependent operations.  As separate kernels each of them pays a launch boundary and a cold start
// of its loads; here the blocks stay resident, a phase begins right behind the barrier, and the
// things between the matrix products cost no pass over memory of their own:
//   * the residual sum and the sum of squares for the next RMS norm are formed in the epilogue of
//     the product that makes the branch output (per-block partial sums, added in a fixed order:
//     deterministic); the norm itself is applied while the next product stages its input;
//   * rotation of q and of the new k, and the write of k, v into their page, happen inside the
//     attention phase; silu(gate) * up is the epilogue of the gate/up product.
//
// Arithmetic follows the separate kernels: float32 accumulation, softmax, norm statistics,
// rotation angles and residual; outputs of products rounded to bfloat16 before they are added or
// activated; the norm casts to bfloat16 before the weight (src/layers/layernorm.py:21-23).
// Formulas: src/models/llama.py:66-89 (block), src/layers/attention.py:35-71,
// src/layers/rotary_embedding.py:29-54, src/layers/activation.py:6-9.
//
// The grid barrier spins on a counter in global memory with a limit on its iterations: when the
// limit is reached the block records status 2 and every later barrier is skipped, so the kernel
// always returns (its results are then void and the host raises).  The launch is cooperative, so
// all blocks are resident and the barrier cannot starve.

#include <cooperative_groups.h>

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int D = HEAD_DIM;
constexpr int THREADS = 512;
constexpr int WARPS = THREADS / 32;
constexpr int KB = 64;                 // k elements per block of a product
constexpr int MT = 16;                 // most tokens
constexpr int NT = MT / 8;             // token tiles of the mma
constexpr int WN = D <= 64 ? 16 : (D <= 128 ? 8 : 4);    // warps that split the keys of a tile
constexpr int KT = 16 * WN;            // keys per attention tile: 16 for each of those warps
constexpr int LDS = D + 8;             // row stride of a key/value tile in shared memory
constexpr long long SPIN_LIMIT = 4LL * 1000 * 1000;      // about two seconds of polling
static_assert(D % 32 == 0 && D >= 32 && D <= 256, "head size must be a multiple of 32 up to 256");

struct LayerPtrs {
    const __nv_bfloat16* w_qkv;        // [(heads + 2 kv_heads) * D, width]
    const __nv_bfloat16* w_o;          // [width, heads * D]
    const __nv_bfloat16* w_gate_up;    // [2 inner, width], gate rows first
    const __nv_bfloat16* w_down;       // [width, inner]
    const void* norm1;                 // [width], bfloat16 or float32
    const void* norm2;
    __nv_bfloat16* k_pages;            // [pages, kv_heads, page, D]
    __nv_bfloat16* v_pages;
};

struct Args {
    const LayerPtrs* layers;
    int num_layers;
    const __nv_bfloat16* embedding;    // [vocab, width]
    const void* final_norm;
    const __nv_bfloat16* lm_head;      // [vocab, width]
    int norm_f32;                      // norm weights are float32 (else bfloat16)
    int width, heads, kv_heads, inner, vocab;
    float eps, scale;
    const float* inv_freq;             // [D / 2]
    const int* block_table;
    int table_stride, page, num_pages;
    int m;                             // tokens (= sequences) of the step
    const int* token_ids;
    const int* positions;              // position of each token = keys already cached
    const int* slots;
    const int* logit_rows;
    int num_logit_rows;
    float* resid_a;                    // [MT, width]
    float* resid_b;
    float* ssq_part;                   // [2 layers + 1][grid][MT] partial sums of squares
    __nv_bfloat16* qkv;                // [MT, (heads + 2 kv_heads) * D]
    __nv_bfloat16* ctx;                // [MT, heads * D]
    __nv_bfloat16* act;                // [MT, inner]
    float* part_acc;                   // [MT * kv_heads * chunks][16][D]
    float* part_ml;                    // [MT * kv_heads * chunks][16][2]
    int chunks, chunk_keys;            // key ranges are cut at multiples of chunk_keys
    float* logits;                     // [num_logit_rows, vocab]
    unsigned* barrier;                 // zeroed before the launch
    int* status;
    unsigned long long* timing;        // optional: [grid][stamps] nanosecond stamps of block phases
    int timing_slots;
};

// ------------------------------------------------------------------------------------------ helpers
__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// data another block wrote before the last barrier: never through the non-coherent path
__device__ __forceinline__ uint4 load_fresh(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 load_fresh_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float load_fresh_f(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned load_fresh_u32(const void* p) {
    unsigned v;
    asm volatile("ld.global.cg.u32 %0, [%1];\n" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float load_fresh_bf16(const __nv_bfloat16* p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];\n" : "=h"(v) : "l"(p));
    return __bfloat162float(__ushort_as_bfloat16(v));
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
__device__ __forceinline__ float bf16_round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(unsigned u) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&u);
    return make_float2(__low2float(v), __high2float(v));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ float norm_weight(const void* w, int f32, int i) {
    return f32 ? reinterpret_cast<const float*>(w)[i]
               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}
// a time stamp of this block (thread 0), when the launch asked for them
__device__ __forceinline__ void stamp(const Args& a, int& slot) {
    if (a.timing != nullptr && threadIdx.x == 0 && slot < a.timing_slots)
        a.timing[(size_t)blockIdx.x * a.timing_slots + slot] = global_ns();
    ++slot;
}

// All blocks of the grid wait for each other.  `target` counts the arrivals expected so far.
__device__ void grid_barrier(const Args& a, unsigned& target, int& slot) {
    __syncthreads();
    stamp(a, slot);                                   // this block's work of the phase is done
    if (threadIdx.x == 0) {
        target += gridDim.x;
        if (load_fresh_u32(a.status) != 2u) {
            __threadfence();
            atomicAdd(a.barrier, 1u);
            long long spins = 0;
            for (;;) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.u32 %0, [%1];\n" : "=r"(seen) : "l"(a.barrier));
                if (seen >= target) break;
                if (++spins > SPIN_LIMIT || load_fresh_u32(a.status) == 2u) {
                    atomicExch(a.status, 2);                     // give up: later barriers are skipped
                    break;
                }
            }
        }
    }
    __syncthreads();
    stamp(a, slot);                                   // the barrier has opened
}

// ------------------------------------------------------------------------------------------ products
// The rows [r_begin, r_end) of out = x w^T for this block, in tiles of 16 rows.  T tiles are worked
// on at a time, each by 16 / T warps that take the 64-wide k blocks of their tile in turn; partial
// sums meet in shared memory.  x comes from shared memory (XS: staged and normalised there) or
// from global memory.  GATED: w stacks n_out gate rows over n_out up rows, and the epilogue gets
// both sums.  TOK: token tiles of 8.  The epilogue runs in thread (slot, token, row) order:
// a thread always serves the same token, (threadIdx.x & 255) >> 4.
template <int T, int TOK, bool GATED, bool XS, typename Epilogue>
__device__ void product_tiles(const __nv_bfloat16* __restrict__ w, int n_out, int k_dim,
                              int r_begin, int r_end, const __nv_bfloat16* x, int ldx, int m_rows,
                              float* red, Epilogue& epilogue) {
    constexpr int SETS = GATED ? 2 : 1;
    constexpr int U = 2;
    constexpr int WPT = WARPS / T;                       // warps per tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int slot = warp / WPT, wk = warp % WPT;
    const int blocks = (k_dim + KB - 1) / KB;
    const int tiles = (r_end - r_begin + 15) / 16;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    float (*red4)[SETS][16][NT * 8 + 1] = reinterpret_cast<float (*)[SETS][16][NT * 8 + 1]>(red);

    for (int base = 0; base < tiles; base += T) {
        const int r0 = r_begin + (base + slot) * 16;
        const __nv_bfloat16* wrow[SETS][2];
        bool wlive[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = r0 + g + 8 * h;
            wlive[h] = r < r_end;
#pragma unroll
            for (int s = 0; s < SETS; ++s)
                wrow[s][h] = w + (size_t)((wlive[h] ? r : r_begin) + s * n_out) * k_dim + 8 * t;
        }
        float acc[SETS][TOK][4];
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < TOK; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[s][j][e] = 0.0f;

        if (r0 < r_end) {                                // this slot has a tile (uniform over the warp)
            for (int b0 = wk; b0 < blocks; b0 += WPT * U) {
                uint4 wv[U][SETS][2][2], xv[U][TOK][2];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int k0 = (b0 + u * WPT) * KB;
                    const bool ok0 = k0 + 8 * t + 8 <= k_dim, ok1 = k0 + 32 + 8 * t + 8 <= k_dim;
#pragma unroll
                    for (int s = 0; s < SETS; ++s)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            wv[u][s][h][0] = (ok0 && wlive[h]) ? load_stream(wrow[s][h] + k0) : zero;
                            wv[u][s][h][1] =
                                (ok1 && wlive[h]) ? load_stream(wrow[s][h] + k0 + 32) : zero;
                        }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int k0 = (b0 + u * WPT) * KB;
                    const bool ok0 = k0 + 8 * t + 8 <= k_dim, ok1 = k0 + 32 + 8 * t + 8 <= k_dim;
#pragma unroll
                    for (int j = 0; j < TOK; ++j) {
                        const int mrow = j * 8 + g;
                        const bool live = mrow < m_rows;
                        const __nv_bfloat16* xp = x + (size_t)(live ? mrow : 0) * ldx + 8 * t + k0;
                        if (XS) {
                            xv[u][j][0] = (ok0 && live) ? *reinterpret_cast<const uint4*>(xp) : zero;
                            xv[u][j][1] =
                                (ok1 && live) ? *reinterpret_cast<const uint4*>(xp + 32) : zero;
                        } else {
                            xv[u][j][0] = (ok0 && live) ? load_fresh(xp) : zero;
                            xv[u][j][1] = (ok1 && live) ? load_fresh(xp + 32) : zero;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int p = 0; p < 2; ++p)
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int s = 0; s < SETS; ++s) {
                                const unsigned a0 = regs(wv[u][s][0][p])[2 * q];
                                const unsigned a2 = regs(wv[u][s][0][p])[2 * q + 1];
                                const unsigned a1 = regs(wv[u][s][1][p])[2 * q];
                                const unsigned a3 = regs(wv[u][s][1][p])[2 * q + 1];
#pragma unroll
                                for (int j = 0; j < TOK; ++j)
                                    mma_bf16(acc[s][j], a0, a1, a2, a3, regs(xv[u][j][p])[2 * q],
                                             regs(xv[u][j][p])[2 * q + 1]);
                            }
            }
        }
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
            for (int j = 0; j < TOK; ++j) {
                red4[warp][s][g][j * 8 + 2 * t] = acc[s][j][0];
                red4[warp][s][g][j * 8 + 2 * t + 1] = acc[s][j][1];
                red4[warp][s][g + 8][j * 8 + 2 * t] = acc[s][j][2];
                red4[warp][s][g + 8][j * 8 + 2 * t + 1] = acc[s][j][3];
            }
        __syncthreads();
        for (int e = threadIdx.x; e < T * 16 * MT; e += THREADS) {
            const int sl = e >> 8, mrow = (e & 255) >> 4, r = e & 15;
            const int row = r_begin + (base + sl) * 16 + r;
            if (mrow < m_rows && row < r_end) {
                float v[SETS];
#pragma unroll
                for (int s = 0; s < SETS; ++s) {
                    float sum = 0.0f;
#pragma unroll
                    for (int wi = 0; wi < WPT; ++wi) sum += red4[sl * WPT + wi][s][r][mrow];
                    v[s] = sum;
                }
                epilogue(mrow, row, v[0], v[SETS - 1]);
            }
        }
        __syncthreads();
    }
}

template <int TOK, bool GATED, bool XS, typename Epilogue>
__device__ void product_rows(const __nv_bfloat16* __restrict__ w, int n_out, int k_dim, int r_begin,
                             int r_end, const __nv_bfloat16* x, int ldx, int m_rows, float* red,
                             Epilogue epilogue) {
    const int tiles = (r_end - r_begin + 15) / 16;       // the same in every thread of the block
    if (tiles >= 3)
        product_tiles<4, TOK, GATED, XS>(w, n_out, k_dim, r_begin, r_end, x, ldx, m_rows, red,
                                         epilogue);
    else if (tiles == 2)
        product_tiles<2, TOK, GATED, XS>(w, n_out, k_dim, r_begin, r_end, x, ldx, m_rows, red,
                                         epilogue);
    else
        product_tiles<1, TOK, GATED, XS>(w, n_out, k_dim, r_begin, r_end, x, ldx, m_rows, red,
                                         epilogue);
}

// x_s[m][:] = bf16( bf16(resid[row(m)][:] * inv_rms[m]) * weight ), inv_rms from the per-block
// partial sums of squares that the previous phase left (added in a fixed order).  The loads of
// the residual are issued first; the sums are fetched and reduced while they are in flight.
__device__ __forceinline__ void norm_weight4(const void* w, int f32, int k, float (&out)[4]) {
    if (f32) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + k);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(w) + k);
        const float2 lo = unpack_bf16(v.x), hi = unpack_bf16(v.y);
        out[0] = lo.x; out[1] = lo.y; out[2] = hi.x; out[3] = hi.y;
    }
}

__device__ void stage_normed(const Args& a, const float* resid, const int* rows, int m_rows,
                             const float* ssq, const void* weight, __nv_bfloat16* x_s, int lds,
                             float* inv_s) {
    const int quads = a.width >> 2, total = m_rows * quads;
    constexpr int B = 8;                                  // loads in flight per thread
    float4 r[B];
    auto load_batch = [&](int base) {
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int idx = base + i * THREADS;
            if (idx < total) {
                const int mrow = idx / quads, k = 4 * (idx - mrow * quads);
                r[i] = load_fresh_f4(resid + (size_t)(rows ? rows[mrow] : mrow) * a.width + k);
            }
        }
    };
    int base = threadIdx.x;
    load_batch(base);
    {
        // warp w adds the partial sums of token w (of token rows[w] when rows are picked): lanes
        // take the blocks in turn, then the lanes' sums are added in a fixed order
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (warp < m_rows) {
            const int tok = rows ? rows[warp] : warp;
            float total_sq = 0.0f;
            for (int c = lane; c < (int)gridDim.x; c += 32)
                total_sq += load_fresh_f(ssq + (size_t)c * MT + tok);
            total_sq = warp_sum(total_sq);
            if (lane == 0) inv_s[warp] = rsqrtf(total_sq / (float)a.width + a.eps);
        }
    }
    __syncthreads();
    for (;;) {
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int idx = base + i * THREADS;
            if (idx < total) {
                const int mrow = idx / quads, k = 4 * (idx - mrow * quads);
                const float inv = inv_s[mrow];
                float w4[4];
                norm_weight4(weight, a.norm_f32, k, w4);
                uint2 packed;
                packed.x = pack_bf16(bf16_round(r[i].x * inv) * w4[0], bf16_round(r[i].y * inv) * w4[1]);
                packed.y = pack_bf16(bf16_round(r[i].z * inv) * w4[2], bf16_round(r[i].w * inv) * w4[3]);
                *reinterpret_cast<uint2*>(x_s + (size_t)mrow * lds + k) = packed;
            }
        }
        base += THREADS * B;
        if (base >= total) break;
        load_batch(base);
    }
    __syncthreads();
}

// After a product whose epilogue summed squares per token in the threads (a thread serves token
// (threadIdx.x & 255) >> 4): one partial per block and token, added in a fixed order.
__device__ void store_ssq(float local, float* ssq_block, int m_rows, float* tmp /* 32 floats */) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 15) == 0) tmp[threadIdx.x >> 4] = local;        // 32 groups of 16 threads
    __syncthreads();
    if (threadIdx.x < m_rows) ssq_block[threadIdx.x] = tmp[threadIdx.x] + tmp[threadIdx.x + 16];
    __syncthreads();
}

// ------------------------------------------------------------------------------------------ attention
// One unit: token m, kv head hk, chunk c of its keys.  The first WN warps each take 16 keys of a
// tile of KT keys (the narrow shape of attention_mma.cu, with more warps), rows are the query
// heads of the group; the remaining warps only load tiles and keep the block's barriers.
__device__ void attention_unit(const Args& a, const LayerPtrs& L, int m, int hk, int c,
                               unsigned char* smem_raw) {
    constexpr int NK = 16, NTS = NK / 8, DT = D / 8, CHUNKS = D / 8;
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* v_s = k_s + 2 * KT * LDS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int g = a.heads / a.kv_heads;
    const int pos = a.positions[m], slot = a.slots[m];
    const int qkv_stride = (a.heads + 2 * a.kv_heads) * D;
    const __nv_bfloat16* row = a.qkv + (size_t)m * qkv_stride;
    const int kv_begin = c * a.chunk_keys;
    const int kv_end = min((c + 1) * a.chunk_keys, pos + 1);
    const bool mine = kv_begin < kv_end;                       // uniform over the block
    const size_t slab = (size_t)a.page * D;

    // the new token's key (rotated) and value go into their page; the chunk that holds the
    // position does it, before it reads its tiles
    if (mine && pos >= kv_begin && pos < kv_end) {
        const int page_id = a.block_table[(size_t)slot * a.table_stride + pos / a.page];
        if (page_id < 0 || page_id >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.status, 1);
        } else {
            const size_t off = ((size_t)page_id * a.kv_heads + hk) * slab + (size_t)(pos % a.page) * D;
            const __nv_bfloat16* kn = row + (size_t)(a.heads + hk) * D;
            const __nv_bfloat16* vn = row + (size_t)(a.heads + a.kv_heads + hk) * D;
            for (int j = threadIdx.x; j < D / 2; j += THREADS) {
                const float ang = (float)pos * a.inv_freq[j];
                const float cs = cosf(ang), sn = sinf(ang);
                const float x1 = load_fresh_bf16(kn + j), x2 = load_fresh_bf16(kn + j + D / 2);
                L.k_pages[off + j] = __float2bfloat16_rn(x1 * cs - x2 * sn);
                L.k_pages[off + j + D / 2] = __float2bfloat16_rn(x2 * cs + x1 * sn);
            }
            for (int j = threadIdx.x; j < D; j += THREADS)
                L.v_pages[off + j] = __float2bfloat16_rn(load_fresh_bf16(vn + j));
        }
    }
    __syncthreads();
    if (!mine) return;                                          // the merge skips empty chunks

    const int tiles_rows = (g + 15) / 16;                       // 16 query heads a pass
    for (int tr = 0; tr < tiles_rows; ++tr) {
        bool live[2];
        int hq[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = tr * 16 + gid + 8 * i;
            live[i] = r < g;
            hq[i] = hk * g + (live[i] ? r : 0);
        }
        unsigned qf[D / 16][4];
        if (warp < WN) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const __nv_bfloat16* p = row + (size_t)hq[i] * D + kk * 16 + 2 * tig;
                    qf[kk][i] = live[i] ? load_fresh_u32(p) : 0u;
                    qf[kk][i + 2] = live[i] ? load_fresh_u32(p + 8) : 0u;
                }
            // rotate: feature j pairs with j + D/2, which sits D/32 k-steps further in this thread
#pragma unroll
            for (int kk = 0; kk < D / 32; ++kk)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int col = kk * 16 + 2 * tig + 8 * half;
                    const float a0 = (float)pos * a.inv_freq[col], a1 = (float)pos * a.inv_freq[col + 1];
                    const float c0 = cosf(a0), s0 = sinf(a0), c1 = cosf(a1), s1 = sinf(a1);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int e = 2 * half + i;
                        const float2 lo = unpack_bf16(qf[kk][e]), hi = unpack_bf16(qf[kk + D / 32][e]);
                        qf[kk][e] = pack_bf16(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
                        qf[kk + D / 32][e] = pack_bf16(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
                    }
                }
        }
        const int k_lo = (kv_begin / KT) * KT;
        auto load_tile = [&](int kt, int stage) {
            __nv_bfloat16* kd = k_s + stage * KT * LDS;
            __nv_bfloat16* vd = v_s + stage * KT * LDS;
            for (int ch = threadIdx.x; ch < KT * CHUNKS; ch += THREADS) {
                const int j = ch / CHUNKS, part = ch - j * CHUNKS;
                const int kpos = kt + j;
                bool ok = kpos >= kv_begin && kpos < kv_end;
                size_t off = 0;
                if (ok) {
                    const int page_id = a.block_table[(size_t)slot * a.table_stride + kpos / a.page];
                    ok = page_id >= 0 && page_id < a.num_pages;
                    if (ok) off = ((size_t)page_id * a.kv_heads + hk) * slab +
                                  (size_t)(kpos % a.page) * D + part * 8;
                }
                cp_async16(kd + j * LDS + part * 8, L.k_pages + off, ok);
                cp_async16(vd + j * LDS + part * 8, L.v_pages + off, ok);
            }
        };
        float o_acc[DT][4];
#pragma unroll
        for (int j = 0; j < DT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.0f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
        const float sl = a.scale * 1.4426950408889634f;

        load_tile(k_lo, 0);
        cp_async_commit();
        int stage = 0;
        for (int kt = k_lo; kt < kv_end; kt += KT, stage ^= 1) {
            if (kt + KT < kv_end) load_tile(kt + KT, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();
            const int key0 = kt + warp * NK;
            if (warp < WN && key0 < kv_end) {
                const __nv_bfloat16* kb = k_s + stage * KT * LDS + warp * NK * LDS;
                const __nv_bfloat16* vb = v_s + stage * KT * LDS + warp * NK * LDS;
                float s[NTS][4];
#pragma unroll
                for (int j = 0; j < NTS; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    unsigned b[4];
                    const int mat = lane >> 3, r = lane & 7;
                    ldmatrix_x4(b, kb + ((mat >> 1) * 8 + r) * LDS + kk * 16 + (mat & 1) * 8);
                    mma_bf16(s[0], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b[0], b[1]);
                    mma_bf16(s[1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b[2], b[3]);
                }
                if (key0 < kv_begin || key0 + NK > kv_end) {
#pragma unroll
                    for (int j = 0; j < NTS; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int key = key0 + j * 8 + 2 * tig + (e & 1);
                            if (key < kv_begin || key >= kv_end) s[j][e] = -INFINITY;
                        }
                }
                float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
                for (int j = 0; j < NTS; ++j) {
                    m_new[0] = fmaxf(m_new[0], fmaxf(s[j][0], s[j][1]));
                    m_new[1] = fmaxf(m_new[1], fmaxf(s[j][2], s[j][3]));
                }
                float corr[2], m_use[2], l_add[2] = {0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
                    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
                    m_use[i] = m_new[i] == -INFINITY ? 0.0f : m_new[i];
                    corr[i] = fast_exp2((m_run[i] - m_use[i]) * sl);
                    m_run[i] = m_new[i];
                }
                unsigned pf[4];
#pragma unroll
                for (int j = 0; j < NTS; ++j) {
                    const float p0 = fast_exp2((s[j][0] - m_use[0]) * sl);
                    const float p1 = fast_exp2((s[j][1] - m_use[0]) * sl);
                    const float p2 = fast_exp2((s[j][2] - m_use[1]) * sl);
                    const float p3 = fast_exp2((s[j][3] - m_use[1]) * sl);
                    l_add[0] += p0 + p1;
                    l_add[1] += p2 + p3;
                    pf[j * 2] = pack_bf16(p0, p1);
                    pf[j * 2 + 1] = pack_bf16(p2, p3);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_add[i];
#pragma unroll
                for (int j = 0; j < DT; ++j) {
                    o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0];
                    o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
                }
#pragma unroll
                for (int jd = 0; jd < DT; jd += 2) {
                    unsigned b[4];
                    const int mat = lane >> 3, r = lane & 7;
                    ldmatrix_x4_trans(b, vb + ((mat & 1) * 8 + r) * LDS + (jd + (mat >> 1)) * 8);
                    mma_bf16(o_acc[jd], pf[0], pf[1], pf[2], pf[3], b[0], b[1]);
                    mma_bf16(o_acc[jd + 1], pf[0], pf[1], pf[2], pf[3], b[2], b[3]);
                }
            }
            __syncthreads();
        }
        cp_async_wait<0>();
        // merge the warps through shared memory
        float* red_o = reinterpret_cast<float*>(smem_raw);                 // [WN][16][D]
        float* red_m = red_o + WN * 16 * D;
        float* red_l = red_m + WN * 16;
        __syncthreads();
        if (warp < WN) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
                const int r = gid + 8 * i;
                float* dst = red_o + ((size_t)warp * 16 + r) * D;
#pragma unroll
                for (int j = 0; j < DT; ++j) {
                    dst[j * 8 + 2 * tig] = o_acc[j][2 * i];
                    dst[j * 8 + 2 * tig + 1] = o_acc[j][2 * i + 1];
                }
                if (tig == 0) {
                    red_m[warp * 16 + r] = m_run[i];
                    red_l[warp * 16 + r] = l_run[i];
                }
            }
        }
        __syncthreads();
        const int unit = (m * a.kv_heads + hk) * a.chunks + c;
        for (int e = threadIdx.x; e < 16 * D; e += THREADS) {
            const int r = e / D, dd = e - r * D;
            const int head_in_group = tr * 16 + r;
            if (head_in_group >= g) continue;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < WN; ++w) mx = fmaxf(mx, red_m[w * 16 + r]);
            float l = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WN; ++w) {
                const float mw = red_m[w * 16 + r];
                if (mw == -INFINITY) continue;
                const float f = fast_exp2((mw - mx) * sl);
                l += red_l[w * 16 + r] * f;
                acc += red_o[((size_t)w * 16 + r) * D + dd] * f;
            }
            if (a.chunks == 1) {
                a.ctx[(size_t)m * a.heads * D + (size_t)(hk * g + head_in_group) * D + dd] =
                    __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
            } else {
                const size_t idx = ((size_t)unit * tiles_rows + tr) * 16 + r;
                a.part_acc[idx * D + dd] = acc;
                if (dd == 0) {
                    a.part_ml[idx * 2] = mx * a.scale;
                    a.part_ml[idx * 2 + 1] = l;
                }
            }
        }
        __syncthreads();
    }
}

// shared memory: [x_s: MT x (width + 8) bf16, also the attention tiles] [red] [inv] [tmp]
__host__ __device__ inline size_t region_bytes(int width) {
    size_t xs = (size_t)MT * (width + 8) * sizeof(__nv_bfloat16);
    const size_t attn = (size_t)4 * KT * LDS * sizeof(__nv_bfloat16);
    const size_t attn_red = (size_t)WN * 16 * (D + 2) * sizeof(float);
    if (attn > xs) xs = attn;
    if (attn_red > xs) xs = attn_red;
    return (xs + 15) & ~(size_t)15;
}
constexpr size_t RED_FLOATS = (size_t)WARPS * 2 * 16 * (NT * 8 + 1);

// ------------------------------------------------------------------------------------------ the kernel
// TOK: token tiles of 8 that the products carry (1 for up to 8 tokens, 2 for up to 16).
template <int TOK>
__global__ void __launch_bounds__(THREADS, 1) decode_fused_kernel(const __grid_constant__ Args a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lds = a.width + 8;
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + region_bytes(a.width));
    float* inv_s = red + RED_FLOATS;
    float* tmp = inv_s + MT;

    const int G = gridDim.x, cta = blockIdx.x;
    const int M = a.m;
    unsigned target = 0;
    int slot = 0;
    stamp(a, slot);
    const int qkv_rows = (a.heads + 2 * a.kv_heads) * D;
    auto share = [&](int n, int& lo, int& hi) {             // this block's rows of n
        lo = (int)((long long)n * cta / G);
        hi = (int)((long long)n * (cta + 1) / G);
    };
    const int my_token = (threadIdx.x & 255) >> 4;           // the token a thread's epilogues serve

    // ---- embedding: residual rows and their sums of squares (this block's columns)
    {
        int lo, hi;
        share(a.width, lo, hi);
        float local = 0.0f;
        if (threadIdx.x < 256 && my_token < M) {
            int id = a.token_ids[my_token];
            if (id < 0 || id >= a.vocab) id = 0;
            for (int k = lo + (threadIdx.x & 15); k < hi; k += 16) {
                const float v = __bfloat162float(a.embedding[(size_t)id * a.width + k]);
                a.resid_a[(size_t)my_token * a.width + k] = v;
                local += v * v;
            }
        }
        store_ssq(local, a.ssq_part + (size_t)cta * MT, M, tmp);
    }
    grid_barrier(a, target, slot);

    for (int layer = 0; layer < a.num_layers; ++layer) {
        const LayerPtrs L = a.layers[layer];
        const float* ssq1 = a.ssq_part + (size_t)(2 * layer) * G * MT;
        float* ssq2 = a.ssq_part + (size_t)(2 * layer + 1) * G * MT;
        float* ssq3 = a.ssq_part + (size_t)(2 * layer + 2) * G * MT;

        // ---- q, k, v = norm(resid_a) w_qkv^T
        {
            int lo, hi;
            share(qkv_rows, lo, hi);
            stage_normed(a, a.resid_a, nullptr, M, ssq1, L.norm1, x_s, lds, inv_s);
            product_rows<TOK, false, true>(
                L.w_qkv, qkv_rows, a.width, lo, hi, x_s, lds, M, red,
                [&](int mrow, int n, float v, float) {
                    a.qkv[(size_t)mrow * qkv_rows + n] = __float2bfloat16_rn(v);
                });
        }
        grid_barrier(a, target, slot);

        // ---- attention over the pages (rotation and cache write inside)
        {
            const int units = M * a.kv_heads * a.chunks;
            for (int u = cta; u < units; u += G) {
                const int c = u % a.chunks, hk = (u / a.chunks) % a.kv_heads;
                attention_unit(a, L, u / (a.chunks * a.kv_heads), hk, c, smem_raw);
            }
        }
        grid_barrier(a, target, slot);
        if (a.chunks > 1) {
            // merge the chunks of every (token, query head): one warp a row
            const int g = a.heads / a.kv_heads, tiles_rows = (g + 15) / 16;
            const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            for (int row = cta * WARPS + warp; row < M * a.heads; row += G * WARPS) {
                const int mrow = row / a.heads, h = row - mrow * a.heads;
                const int hk = h / g, r = h - hk * g;
                const int n = a.positions[mrow] / a.chunk_keys + 1;      // chunks that hold keys
                float mx = -INFINITY;
                for (int c = 0; c < n; ++c) {
                    const size_t idx = ((size_t)((mrow * a.kv_heads + hk) * a.chunks + c) * tiles_rows +
                                        r / 16) * 16 + r % 16;
                    mx = fmaxf(mx, load_fresh_f(a.part_ml + idx * 2));
                }
                float l = 0.0f, acc[D / 32];
#pragma unroll
                for (int i = 0; i < D / 32; ++i) acc[i] = 0.0f;
                for (int c = 0; c < n; ++c) {
                    const size_t idx = ((size_t)((mrow * a.kv_heads + hk) * a.chunks + c) * tiles_rows +
                                        r / 16) * 16 + r % 16;
                    const float mc = load_fresh_f(a.part_ml + idx * 2);
                    if (mc == -INFINITY) continue;
                    const float f = expf(mc - mx);
                    l += load_fresh_f(a.part_ml + idx * 2 + 1) * f;
#pragma unroll
                    for (int i = 0; i < D / 32; ++i)
                        acc[i] = fmaf(load_fresh_f(a.part_acc + idx * D + lane + 32 * i), f, acc[i]);
                }
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
                for (int i = 0; i < D / 32; ++i)
                    a.ctx[(size_t)mrow * a.heads * D + (size_t)h * D + lane + 32 * i] =
                        __float2bfloat16_rn(acc[i] * inv);
            }
            grid_barrier(a, target, slot);
        }

        // ---- resid_b = resid_a + ctx w_o^T, and its sums of squares
        {
            int lo, hi;
            share(a.width, lo, hi);
            float local = 0.0f;
            product_rows<TOK, false, false>(
                L.w_o, a.width, a.heads * D, lo, hi, a.ctx, a.heads * D, M, red,
                [&](int mrow, int n, float v, float) {
                    const float r = load_fresh_f(a.resid_a + (size_t)mrow * a.width + n) + bf16_round(v);
                    a.resid_b[(size_t)mrow * a.width + n] = r;
                    local += r * r;
                });
            store_ssq(local, ssq2 + (size_t)cta * MT, M, tmp);
        }
        grid_barrier(a, target, slot);

        // ---- act = silu(gate) * up of norm(resid_b)
        {
            int lo, hi;
            share(a.inner, lo, hi);
            stage_normed(a, a.resid_b, nullptr, M, ssq2, L.norm2, x_s, lds, inv_s);
            product_rows<TOK, true, true>(
                L.w_gate_up, a.inner, a.width, lo, hi, x_s, lds, M, red,
                [&](int mrow, int n, float gate, float up) {
                    const float gr = bf16_round(gate), ur = bf16_round(up);
                    a.act[(size_t)mrow * a.inner + n] = __float2bfloat16_rn(gr / (1.0f + expf(-gr)) * ur);
                });
        }
        grid_barrier(a, target, slot);

        // ---- resid_a = resid_b + act w_down^T, and its sums of squares
        {
            int lo, hi;
            share(a.width, lo, hi);
            float local = 0.0f;
            product_rows<TOK, false, false>(
                L.w_down, a.width, a.inner, lo, hi, a.act, a.inner, M, red,
                [&](int mrow, int n, float v, float) {
                    const float r = load_fresh_f(a.resid_b + (size_t)mrow * a.width + n) + bf16_round(v);
                    a.resid_a[(size_t)mrow * a.width + n] = r;
                    local += r * r;
                });
            store_ssq(local, ssq3 + (size_t)cta * MT, M, tmp);
        }
        grid_barrier(a, target, slot);
    }

    // ---- logits = norm(resid_a[rows]) w_lm^T
    if (a.num_logit_rows > 0) {
        int lo, hi;
        share(a.vocab, lo, hi);
        const float* ssq_last = a.ssq_part + (size_t)(2 * a.num_layers) * G * MT;
        stage_normed(a, a.resid_a, a.logit_rows, a.num_logit_rows, ssq_last, a.final_norm, x_s, lds,
                     inv_s);
        product_rows<TOK, false, true>(a.lm_head, a.vocab, a.width, lo, hi, x_s, lds,
                                       a.num_logit_rows, red, [&](int r, int n, float v, float) {
                                           a.logits[(size_t)r * a.vocab + n] = v;
                                       });
    }
    stamp(a, slot);
}

size_t shared_bytes(int width) {
    return region_bytes(width) + (RED_FLOATS + MT + 32) * sizeof(float);
}

template <int TOK>
int prepare_kernel(size_t smem) {
    return (int)cudaFuncSetAttribute(decode_fused_kernel<TOK>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

}  // namespace

DE_EXPORT int de_decode_fused_head_dim() { return D; }
DE_EXPORT int de_decode_fused_max_tokens() { return MT; }
DE_EXPORT int de_decode_fused_args_bytes() { return (int)sizeof(Args); }
DE_EXPORT int de_decode_fused_layer_bytes() { return (int)sizeof(LayerPtrs); }

// How many blocks the launch uses on the current device (one per SM), or a negative code when the
// kernel cannot be resident with this width.
DE_EXPORT int de_decode_fused_grid(int width) {
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    const size_t smem = shared_bytes(width);
    if (smem > 220 * 1024) return -2;
    if (prepare_kernel<1>(smem) != 0 || prepare_kernel<2>(smem) != 0) return -3;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel<2>, THREADS,
                                                      smem) != cudaSuccess) return -4;
    if (per_sm < 1) return -5;
    return sms;
}

// `args` points to a host copy of Args (the layout is this file's; the Python side fills it with
// ctypes and checks its size against de_decode_fused_args_bytes).
DE_EXPORT int de_decode_fused(const void* args, int grid, void* stream) {
    Args a = *reinterpret_cast<const Args*>(args);
    if (a.m <= 0) return 0;
    if (a.m > MT || a.num_logit_rows > MT || a.width % 8 != 0 || a.inner % 8 != 0 ||
        (a.heads * D) % 8 != 0 || a.heads % a.kv_heads != 0 || a.chunks < 1)
        return -2;
    const size_t smem = shared_bytes(a.width);
    const bool one = a.m <= 8 && a.num_logit_rows <= 8;
    const int set = one ? prepare_kernel<1>(smem) : prepare_kernel<2>(smem);
    if (set != 0) return set;
    void* params[] = {&a};
    const void* kernel = one ? (const void*)decode_fused_kernel<1> : (const void*)decode_fused_kernel<2>;
    return de_check(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(THREADS), params, smem,
                                                (cudaStream_t)stream));
}

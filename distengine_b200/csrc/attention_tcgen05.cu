// Attention over the paged cache for prompt portions on the 5th-generation tensor cores
// (tcgen05.mma with accumulators in tensor memory, TMA page loads), bfloat16, head size 64.
//
// A work item is 256 query rows of one sequence and one kv head (rows are (token, query head of
// the group)) with a range of key positions.  A block owns it as two tiles of 128 rows, A and B,
// that share every tile of 128 keys the block fetches.  Warps:
//   * warps 0-3 are the softmax threads of tile A, warps 4-7 those of tile B: one thread per row
//     (row i of a tile is lane i of tensor memory);
//   * warp 8, one thread, issues the tensor-core work: s = q k^T (four tcgen05.mma M 128, N 128,
//     K 16 per tile, accumulator in tensor memory) and o += p v (eight tcgen05.mma M 128, N 64,
//     K 16, with v as the "MN-major" operand, i.e. exactly as the cache stores it,
//     [key][feature]; o stays in tensor memory for the whole item);
//   * warp 9 fetches the K and V pages of the key tiles (one TMA box per page, 128-byte swizzle,
//     straight from the page pool through the block table), three tiles in flight.
// For every key tile a softmax thread reads its row of s (128 values, tcgen05.ld) into registers,
// tells the tensor-core thread that the columns are free (the scores of the next key tile are
// then computed while this one is still being worked on), finds the row maximum and writes
// p = exp2(...) as bfloat16 into shared memory in the operand layout.  The two row tiles go at
// their own pace: the tensor-core thread polls what each is waiting for.  The running maximum a row's exponentials refer to is only raised when the true
// maximum has grown by more than 2^8 since (then the row of o in tensor memory and the running
// sum are rescaled); in between, values up to 2^8 are exact enough in float32 and in bfloat16's
// range, and the quotient o / l does not depend on the reference.
//
// Formulas as in src/layers/attention.py:35-71 (scale after the product, causal mask, float32
// softmax), grouped-query heads share the kv head's tiles.  Split key ranges write partial
// results in the layout `de_attn_combine` merges.
//
// Every mbarrier wait is bounded (status 3, the block then runs to its end and frees its tensor
// memory); no cluster launch, every block fetches its own tiles.  One block per SM (193 KB of
// shared memory).

#include <cuda.h>

#include "common.cuh"
#include "tensor_maps.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
constexpr int D = HEAD_DIM;            // head size: 64 or 128
static_assert(D == 64 || D == 128, "the tcgen05 attention is built for head sizes 64 and 128");
constexpr int KS = D / 64;             // 64-feature sub-tiles of a row (128 bytes = a swizzle row)
constexpr int TILE_ROWS = 128;         // query rows of a row tile = lanes of tensor memory
constexpr int NROW = D == 64 ? 2 : 1;  // row tiles of a work item (what shared memory has room for)
constexpr int ROWS = NROW * TILE_ROWS; // query rows of a work item
constexpr int KT = 128;                // keys per tile
constexpr int SOFTMAX_WARPS = 4 * NROW;
constexpr int MMA_WARP = SOFTMAX_WARPS, COPY_WARP = SOFTMAX_WARPS + 1;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr int STAGES = D == 64 ? 3 : 2;   // key/value tiles in flight
constexpr int TILE_BYTES = 128 * 128;  // a sub-tile: 128 rows of 128 bytes
constexpr int TMEM_COLS = 512;         // s of row tile x at 128 x; o of row tile x at 256 + D x
constexpr unsigned SPIN_LIMIT = 20u * 1000u * 1000u;
// q of each row tile (KS sub-tiles), STAGES x (k, v) (KS sub-tiles each), p of each row tile (two
// sub-tiles of 64 keys), barriers
constexpr int SMEM_BYTES = (NROW * KS + 2 * STAGES * KS + 2 * NROW) * TILE_BYTES + 256;
constexpr float RESCALE_AFTER = 8.0f;  // raise a row's reference maximum when it lags by 2^8

struct WorkItem {
    int seq, row0, kv_begin, kv_end, partial, pad0, pad1, pad2;
};

// ---------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* status) {
    const unsigned addr = smem_u32(bar);
    for (unsigned spins = 0; spins < SPIN_LIMIT; ++spins) {
        unsigned done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    atomicExch(status, 3);
    return false;
}
// Whether the phase with the given parity is complete; does not wait.
__device__ __forceinline__ bool mbar_test(void* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, void* bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(void* smem_result, unsigned columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void umma_bf16(unsigned d_tmem, unsigned long long a_desc,
                                          unsigned long long b_desc, unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((unsigned)accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_wait_loads() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_load_32cols(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_store_32cols(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_stores() {
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem),
                 "r"(bytes));
}
#ifdef ATTN_TIMING
// Debugging aid, compiled on request only: wall-clock stamps of one block's phases.
__device__ unsigned long long attn_stamps[2 * 64 * 8];
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
#define STAMP(who, tile, k)                                                                  \
    do {                                                                                     \
        if (blockIdx.x == ATTN_TIMING && (tile) < 64)                                        \
            attn_stamps[((who) * 64 + (tile)) * 8 + (k)] = global_ns();                      \
    } while (0)
#else
#define STAMP(who, tile, k) do { } while (0)
#endif
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// K-major operand tile of rows x 64 bfloat16, 128-byte swizzle: groups of 8 rows are 1024 bytes
// apart (stride byte offset); see gemm_tcgen05.cu for the bit fields.
__device__ __forceinline__ unsigned long long desc_k_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// MN-major operand: the tile is stored [k][64 contiguous n] (v as the cache holds it: [key][feature]),
// 128-byte swizzle; groups of 8 k are 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_mn_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3FFFF) >> 4);
#if V_DESC_SWAP
    d |= (unsigned long long)(1024 >> 4) << 16;
    d |= (unsigned long long)1 << 32;
#else
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
#endif
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 operands, a K-major, b K-major or
// MN-major (bit 16), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr unsigned instr_desc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_tcgen05_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                    int out_stride, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                    int table_stride, int num_pages, const int* __restrict__ seq_slot,
                    const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                    const int* __restrict__ seq_pos0, const WorkItem* __restrict__ items,
                    float* __restrict__ partial_acc, float* __restrict__ partial_ml, int heads,
                    int kv_heads, int page, float scale, int window, int* status) {
    // All shared memory is dynamic and starts at the block's window (1024-byte aligned, which the
    // swizzled tiles need; checked below).
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* q_s = smem_raw;                               // [NROW][KS] sub-tiles
    unsigned char* k_s = q_s + NROW * KS * TILE_BYTES;           // [STAGES][KS] sub-tiles
    unsigned char* v_s = k_s + STAGES * KS * TILE_BYTES;         // [STAGES][KS] sub-tiles
    unsigned char* p_s = v_s + STAGES * KS * TILE_BYTES;         // [NROW][2] sub-tiles (128 x 64 keys)
    unsigned long long* bars =
        reinterpret_cast<unsigned long long*>(p_s + 2 * NROW * TILE_BYTES);
    unsigned long long* kv_full = bars;                          // [STAGES] pages of a tile have landed
    unsigned long long* kv_free = bars + STAGES;                 // [STAGES] the tile has been multiplied
    unsigned long long* s_done = bars + 2 * STAGES;              // [2] scores of A / B are complete
    unsigned long long* p_ready = bars + 2 * STAGES + 2;         // [2] p of A / B is written (128 arrivals)
    unsigned long long* o_done = bars + 2 * STAGES + 4;          // [2] p v of A / B is complete
    unsigned long long* s_free = bars + 2 * STAGES + 6;          // [2] s of A / B is in registers (128 arrivals)
    unsigned& tmem_slot = *reinterpret_cast<unsigned*>(bars + 2 * STAGES + 8);

    // blocks are numbered item-major, so that the items run in the order the host gave them
    const WorkItem it = items[blockIdx.x / kv_heads];
    if (it.kv_begin >= it.kv_end || (smem_u32(smem_raw) & 1023u) != 0) {   // padding item
        if ((smem_u32(smem_raw) & 1023u) != 0 && threadIdx.x == 0) atomicExch(status, 4);
        pdl_wait();
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool softmax_thread = warp < SOFTMAX_WARPS;
    const int x = softmax_thread ? warp >> 2 : 0;                // row tile: 0 = A, 1 = B
    const int rowi = (warp & 3) * 32 + lane;                     // row within the row tile
    const int hk = blockIdx.x % kv_heads;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_free[i], 1);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_done[i], 1);
            mbar_init(&p_ready[i], TILE_ROWS);
            mbar_init(&o_done[i], 1);
            mbar_init(&s_free[i], TILE_ROWS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(&tmem_slot, TMEM_COLS);

    // key range of the item and of each row tile: tile t holds the keys k_lo + 128 t .. + 127
    int k_lo_true = it.kv_begin;
    if (window > 0) k_lo_true = max(k_lo_true, pos0 + it.row0 / g - window + 1);
    const int k_lo = (k_lo_true / KT) * KT;
    int n_of[2], k_hi_of[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int first = it.row0 + i * TILE_ROWS;
        n_of[i] = 0;
        k_hi_of[i] = k_lo;
        if (i < NROW && first < rows_total) {
            const int last_row = min(first + TILE_ROWS, rows_total) - 1;
            k_hi_of[i] = min(it.kv_end, pos0 + last_row / g + 1);
            n_of[i] = max(0, (k_hi_of[i] - k_lo + KT - 1) / KT);
        }
    }
    const int n_tiles = max(n_of[0], n_of[1]);
    const int k_hi = max(k_hi_of[0], k_hi_of[1]);               // beyond it nothing is read

    // this thread's row
    const int r = it.row0 + x * TILE_ROWS + rowi;
    const bool live = softmax_thread && r < rows_total;
    const int tok = live ? r / g : 0;
    const int hq = hk * g + (live ? r % g : 0);
    const int pos = live ? pos0 + tok : -1;
    int lo = it.kv_begin;
    if (window > 0) lo = max(lo, pos - window + 1);
    const int hi = min(it.kv_end, pos + 1);                      // dead row: nothing visible

    pdl_wait();            // q, and the keys and values of this step's tokens, are just written

    // q rows into shared memory, operand layout (chunk index xor row % 8)
    if (softmax_thread) {
        const __nv_bfloat16* src = q + (size_t)(tok0 + tok) * q_stride + hq * D;
        unsigned char* dst = q_s + x * KS * TILE_BYTES + rowi * 128;
#pragma unroll
        for (int c = 0; c < D / 8; ++c)           // chunk c: sub-tile c / 8, place (c % 8) xor row
            cp_async16(dst + (c >> 3) * TILE_BYTES + (((c & 7) ^ (rowi & 7)) << 4), src + c * 8,
                       live);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> tensor core
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem = tmem_slot;
    const float sl = scale * 1.4426950408889634f;
    bool ok = true;

    if (warp == COPY_WARP) {
        // ------------------------------------------------------------------ copies
        const int pages_per_tile = KT / page;
        const unsigned page_bytes = (unsigned)page * 128u;
        int id[4];
        // the pages of a tile that hold keys of the range; the lanes take the pages in turn, so
        // their block-table reads run side by side
        auto lookup = [&](int tile) {
            const int kt = k_lo + tile * KT;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int p = lane + 32 * i;
                const int first = kt + p * page;
                id[i] = -1;
                if (p < pages_per_tile && first + page > k_lo_true && first < k_hi) {
                    id[i] = block_table[(size_t)slot * table_stride + first / page];
                    if (id[i] >= num_pages) id[i] = -1;
                    if (id[i] < 0) atomicExch(status, 2);            // visible keys have no page
                }
            }
        };
        // a TMA box per page; lane 0 announces the bytes
        auto issue = [&](int stage) {
            unsigned bytes = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (id[i] >= 0) bytes += 2 * KS * page_bytes;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, o);
            if (lane == 0) mbar_expect_tx(&kv_full[stage], bytes);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (id[i] < 0) continue;
                const int p = lane + 32 * i;
                const int y = (id[i] * kv_heads + hk) * page;
#pragma unroll
                for (int sub = 0; sub < KS; ++sub) {          // 64 features a box
                    tma_load_2d(k_s + (stage * KS + sub) * TILE_BYTES + p * page_bytes, &map_k,
                                &kv_full[stage], 64 * sub, y);
                    tma_load_2d(v_s + (stage * KS + sub) * TILE_BYTES + p * page_bytes, &map_v,
                                &kv_full[stage], 64 * sub, y);
                }
            }
        };
        for (int t = 0; t < STAGES && t < n_tiles; ++t) {
            lookup(t);
            issue(t);
        }
        for (int tile = STAGES; tile < n_tiles; ++tile) {
            lookup(tile);
            // the stage is free when the tile that used it has been multiplied
            if (ok) ok = mbar_wait(&kv_free[tile % STAGES], ((tile / STAGES) - 1) & 1, status);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) issue(tile % STAGES);
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ tensor core
        constexpr unsigned idesc_s = instr_desc(128, 128, false);
        constexpr unsigned idesc_o = instr_desc(128, 64, true);
        if (lane == 0) {
            // s of row tile i for key tile `tile` (its pages have landed: checked by the caller)
            auto issue_scores = [&](int i, int tile) {
                if (ok) {
#pragma unroll
                    for (int sub = 0; sub < KS; ++sub) {
                        const unsigned long long a = desc_k_major(q_s + (i * KS + sub) * TILE_BYTES);
                        const unsigned long long b =
                            desc_k_major(k_s + ((tile % STAGES) * KS + sub) * TILE_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_bf16(tmem + 128 * i, a + 2 * k, b + 2 * k, idesc_s, sub > 0 || k > 0);
                    }
                }
                umma_commit(&s_done[i]);
            };
            auto wait_tile = [&](int tile) {
                if (ok) ok = mbar_wait(&kv_full[tile % STAGES], (tile / STAGES) & 1, status);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            };
            if (n_tiles > 0) wait_tile(0);
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (n_of[i] > 0) issue_scores(i, 0);
            // The two row tiles go at their own pace: this thread polls what each of them is
            // waiting for and issues whatever has become possible -
            //   the scores of a row tile's next key tile, once its threads hold the current
            //   scores in registers and the key tile has landed;
            //   o += p v, once its threads have written p;
            // and hands a stage back to the copy warp when both row tiles' products that read it
            // are issued.  A poll that finds nothing to do counts towards the iteration limit.
            int s_next[2] = {1, 1}, pv_next[2] = {0, 0};
            int freed = 0;
            unsigned idle = 0;
            while (ok) {
                bool progress = false, busy = false;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (pv_next[i] < n_of[i]) {
                        busy = true;
                        const int tile = pv_next[i];
                        if (mbar_test(&p_ready[i], tile & 1)) {
                            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                            const unsigned long long pa = desc_k_major(p_s + 2 * i * TILE_BYTES);
#pragma unroll
                            for (int sub = 0; sub < KS; ++sub) {      // 64 output features at a time
                                const unsigned long long vb = desc_mn_major(
                                    v_s + ((tile % STAGES) * KS + sub) * TILE_BYTES);
#pragma unroll
                                for (int k = 0; k < KT / 16; ++k) {
                                    // 16 keys of p are 32 bytes inside a sub-tile row (the second
                                    // sub-tile one tile further); 16 keys of v are 2 groups of 8
                                    // rows = 2048 bytes
                                    umma_bf16(tmem + 256 + D * i + 64 * sub,
                                              pa + (unsigned long long)((k >> 2) * (TILE_BYTES >> 4) +
                                                                        2 * (k & 3)),
                                              vb + (unsigned long long)(k * 2048 >> 4), idesc_o,
                                              tile > 0 || k > 0);
                                }
                            }
                            umma_commit(&o_done[i]);
                            STAMP(1, tile, 1 + 2 * i);
                            ++pv_next[i];
                            progress = true;
                        }
                    }
                    if (s_next[i] < n_of[i]) {
                        const int tile = s_next[i];
                        if (mbar_test(&s_free[i], (tile - 1) & 1) &&
                            mbar_test(&kv_full[tile % STAGES], (tile / STAGES) & 1)) {
                            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                            issue_scores(i, tile);
                            STAMP(1, tile, 2 * i);
                            ++s_next[i];
                            progress = true;
                        }
                    }
                }
                while (freed < n_tiles && (freed >= n_of[0] || pv_next[0] > freed) &&
                       (freed >= n_of[1] || pv_next[1] > freed)) {
                    umma_commit(&kv_free[freed % STAGES]);
                    ++freed;
                    progress = true;
                }
                if (!busy) break;
                if (progress) {
                    idle = 0;
                } else if (++idle > SPIN_LIMIT) {
                    atomicExch(status, 3);
                    ok = false;
                }
            }
        }
        __syncwarp();
    } else if (n_of[x] > 0) {
        // ------------------------------------------------------------------ softmax threads
        const unsigned lane_bits = (unsigned)((warp & 3) * 32) << 16;
        const unsigned s_addr = tmem + 128 * x + lane_bits;
        const unsigned o_addr = tmem + 256 + D * x + lane_bits;
        unsigned char* p_row = p_s + 2 * x * TILE_BYTES + rowi * 128;
        const int n_mine = n_of[x];
        float m_ref = -INFINITY;                 // what the exponentials refer to
        float l_run = 0.0f;
        for (int tile = 0; tile < n_mine; ++tile) {
            const int stage = tile % STAGES;
            const int kt = k_lo + tile * KT;
            if (tid == 0) STAMP(0, tile, 0);
            if (ok) ok = mbar_wait(&s_done[x], tile & 1, status);
            if (tid == 0) STAMP(0, tile, 1);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            // only the tiles at the edges of the visible range (the diagonal, a window's start,
            // the first chunk) have keys to hide; the warp decides together
            const bool masked = __any_sync(0xffffffffu, kt < lo || kt + KT > hi);
            // ---- the row of s: 128 values, read once
            unsigned sv[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_load_32cols(s_addr + 32 * c, sv[c]);
            tmem_wait_loads();
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(&s_free[x]);               // the next scores may overwrite these columns
            if (masked) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = kt + 32 * c + i;
                        if (key < lo || key >= hi) sv[c][i] = 0xff800000u;     // -inf
                    }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(sv[c][i]));
            const float m_tile = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            if (tid == 0) STAMP(0, tile, 2);
            // ---- raise the reference where the maximum has run away from it.  That rescales o,
            // which must be at rest: the previous tile's product is waited for first.  Otherwise
            // (nearly always) the exponentials below are formed before that wait: only p's
            // buffer needs the product to be over, not the arithmetic.
            const bool raise = m_tile > m_ref && (m_ref == -INFINITY ||
                                                  (m_tile - m_ref) * sl > RESCALE_AFTER);
            bool o_at_rest = tile == 0;
            if (tile > 0 && __any_sync(0xffffffffu, raise && m_ref != -INFINITY)) {
                if (ok) ok = mbar_wait(&o_done[x], (tile - 1) & 1, status);
                o_at_rest = true;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const float f = (raise && m_ref != -INFINITY) ? fast_exp2((m_ref - m_tile) * sl) : 1.0f;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    unsigned ov[32];
                    tmem_load_32cols(o_addr + 32 * c, ov);
                    tmem_wait_loads();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
                    tmem_store_32cols(o_addr + 32 * c, ov);
                }
                tmem_wait_stores();
                l_run *= f;
            }
            if (raise) m_ref = m_tile;
            // ---- p = exp2((s - reference) sl) as bfloat16 into the operand layout: row rowi of
            // sub-tile (key / 64), 16-byte chunk ((key % 64) / 8) xor (rowi % 8)
            const float m_off = m_ref == -INFINITY ? 0.0f : -m_ref * sl;
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint4 pu[16];                        // the row of p, packed (in place of the scores)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    float p[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        p[j] = fast_exp2(fmaf(__uint_as_float(sv[c][i + j]), sl, m_off));
                        l4[j & 3] += p[j];
                    }
                    uint4 u;
                    u.x = pack2(p[0], p[1]); u.y = pack2(p[2], p[3]);
                    u.z = pack2(p[4], p[5]); u.w = pack2(p[6], p[7]);
                    pu[c * 4 + i / 8] = u;
                }
            }
            l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            // p of the previous tile has been multiplied: its buffer is free
            if (!o_at_rest && ok) ok = mbar_wait(&o_done[x], (tile - 1) & 1, status);
            if (tid == 0) STAMP(0, tile, 3);
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    const int chunk = ((32 * c + i) & 63) >> 3;
                    *reinterpret_cast<uint4*>(p_row + (c >> 1) * TILE_BYTES +
                                              ((chunk ^ (rowi & 7)) << 4)) = pu[c * 4 + i / 8];
                }
            if (tid == 0) STAMP(0, tile, 4);
            // Pages come whole: rows of v beyond the range (the rest of the last page, or keys
            // before a window) may hold anything, and 0 * NaN is NaN in the product.  Row rowi of
            // the stage is key kt + rowi: zero it when it lies outside the item's range.  (Both
            // row tiles do this; they write the same zeros.)
            if (kt + rowi >= k_hi || kt + rowi < k_lo_true) {
                if (ok) ok = mbar_wait(&kv_full[stage], (tile / STAGES) & 1, status);
#pragma unroll
                for (int sub = 0; sub < KS; ++sub) {
                    uint4* vrow = reinterpret_cast<uint4*>(v_s + (stage * KS + sub) * TILE_BYTES +
                                                           rowi * 128);
#pragma unroll
                    for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(&p_ready[x]);
            if (tid == 0) STAMP(0, tile, 5);
        }
        // ---- the item's last product, then the row goes out
        if (ok) ok = mbar_wait(&o_done[x], (n_mine - 1) & 1, status);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        pdl_trigger();
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            unsigned ov[32];
            tmem_load_32cols(o_addr + 32 * c, ov);
            tmem_wait_loads();
            if (!ok || !live) continue;
            if (it.partial < 0) {
                __nv_bfloat16* o = out + (size_t)(tok0 + tok) * out_stride + hq * D + 32 * c;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 u;
                    u.x = pack2(__uint_as_float(ov[j]) * inv, __uint_as_float(ov[j + 1]) * inv);
                    u.y = pack2(__uint_as_float(ov[j + 2]) * inv, __uint_as_float(ov[j + 3]) * inv);
                    u.z = pack2(__uint_as_float(ov[j + 4]) * inv, __uint_as_float(ov[j + 5]) * inv);
                    u.w = pack2(__uint_as_float(ov[j + 6]) * inv, __uint_as_float(ov[j + 7]) * inv);
                    *reinterpret_cast<uint4*>(o + j) = u;
                }
            } else {
                const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + x * TILE_ROWS + rowi;
                float* pa = partial_acc + idx * D + 32 * c;
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(pa + j) =
                        make_float4(__uint_as_float(ov[j]), __uint_as_float(ov[j + 1]),
                                    __uint_as_float(ov[j + 2]), __uint_as_float(ov[j + 3]));
                if (c == 0) {
                    partial_ml[idx * 2] = m_ref * scale;          // natural-log domain, as merged
                    partial_ml[idx * 2 + 1] = l_run;
                }
            }
        }
    } else if (live && it.partial >= 0) {
        // a row tile without a key in this chunk: an empty partial result
        const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + x * TILE_ROWS + rowi;
        for (int j = 0; j < D; ++j) partial_acc[idx * D + j] = 0.0f;
        partial_ml[idx * 2] = -INFINITY;
        partial_ml[idx * 2 + 1] = 0.0f;
    } else if (live) {
        // no key at all for this row (cannot happen for a causal row, whose own key is visible)
        __nv_bfloat16* o = out + (size_t)(tok0 + tok) * out_stride + hq * D;
        for (int j = 0; j < D; ++j) o[j] = __float2bfloat16_rn(0.0f);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------------------------- host side
// the pages of one layer as a matrix [pages * kv_heads * page, 64], boxes of one page
int make_page_map(CUtensorMap* map, const void* pages, long long rows, int page) {
    return tensor_maps::get(map, pages, rows, D, D, page, 64);
}

}  // namespace

#ifdef ATTN_TIMING
DE_EXPORT int de_attn_tcgen05_stamps(unsigned long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, attn_stamps, sizeof(attn_stamps));
}
#endif
DE_EXPORT int de_attn_tcgen05_rows() { return ROWS; }
DE_EXPORT int de_attn_tcgen05_head_dim() { return D; }

// Arguments as de_attn_mma (wide shape); `status` receives 3 if a wait inside the kernel ran out.
DE_EXPORT int de_attn_tcgen05(const void* q, int q_stride, void* out, int out_stride,
                              const void* k_pages, const void* v_pages, const int* block_table,
                              int table_stride, int num_pages, const int* seq_slot,
                              const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                              const int* items, int num_items, float* partial_acc,
                              float* partial_ml, int heads, int kv_heads, int head_dim, int page,
                              float scale, int window, int* status, void* stream) {
    if (num_items <= 0) return 0;
    if (head_dim != D || heads % kv_heads != 0) return -2;
    if (page <= 0 || KT % page != 0 || KT / page > 128 || q_stride % 8 != 0 || out_stride % 8 != 0 ||
        ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)k_pages & 15) ||
        ((uintptr_t)v_pages & 15))
        return -3;
    CUtensorMap map_k, map_v;
    const long long rows = (long long)num_pages * kv_heads * page;
    int code = make_page_map(&map_k, k_pages, rows, page);
    if (code) return code;
    code = make_page_map(&map_v, v_pages, rows, page);
    if (code) return code;
    const size_t smem = SMEM_BYTES;
    static bool sized = false;                 // the attribute is set once
    if (!sized) {
        cudaError_t e = cudaFuncSetAttribute(attn_tcgen05_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        sized = true;
    }
    dim3 grid((unsigned)num_items * (unsigned)kv_heads);
    return de_launch(attn_tcgen05_kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream,
                     (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, map_k, map_v,
                     block_table, table_stride, num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0,
                     (const WorkItem*)items, partial_acc, partial_ml, heads, kv_heads, page, scale,
                     window, status);
}

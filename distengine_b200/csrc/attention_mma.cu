// Attention over the paged cache on the tensor cores, bfloat16 operands, float32 accumulation and
// softmax.  Compiled once per head size (-DHEAD_DIM=d, d a multiple of 16 up to 256), so a run
// compiles the head size of its model only.
//
// The same work items as the float32 kernel (attention_simt.cu): a tile of query rows of one
// sequence and one kv head, rows being (token, query head in the kv head's group), with a range of
// key positions; grouped-query heads share every key/value tile that is loaded
// (the reference expands k and v in memory instead, src/layers/attention.py:35-36).
// Two shapes of one kernel body:
//   wide   - 64 rows: 4 warps x 16 rows, every warp sees all 64 keys of a tile (prompt portions);
//   narrow - 16 rows: 4 warps split the 64 keys of a tile among them and merge at the end
//            (decoded tokens: few rows, long key ranges).
// Keys and values come from the pages through the block table with cp.async (16 bytes a copy,
// zero fill outside the item's range), two tiles in flight; q k^T and p v are mma.sync m16n8k16;
// the softmax is the running maximum / sum form in float32 (exp2 with the scale folded in), masks
// as in src/layers/attention.py:41-64 plus an optional window.  An item that covers a chunk of a
// long key range writes an unnormalised partial (accumulator, maximum, sum) in the layout that
// `de_attn_combine` merges.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int D = HEAD_DIM;
constexpr int KT = 64;                 // keys per tile
constexpr int LDS = D + 8;             // shared-memory row stride in elements: conflict-free ldmatrix
constexpr int THREADS = 128;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");

struct WorkItem {
    int seq, row0, kv_begin, kv_end, partial, pad0, pad1, pad2;
};

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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                         unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {          // ex2.approx: exp2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// WM warps along the rows (16 rows each), WN warps along the keys of a tile; WM * WN = 4.
template <int WM, int WN>
__global__ void __launch_bounds__(THREADS)
attn_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                int out_stride, const __nv_bfloat16* __restrict__ k_pages,
                const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                int table_stride, int num_pages, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                const int* __restrict__ seq_pos0, const WorkItem* __restrict__ items,
                float* __restrict__ partial_acc, float* __restrict__ partial_ml, int heads,
                int kv_heads, int page, float scale, int window) {
    constexpr int ROWS = WM * 16;          // rows of the tile
    constexpr int NK = KT / WN;            // keys of a tile that one warp sees
    constexpr int NT = NK / 8;             // score tiles (n = 8) per warp
    constexpr int DT = D / 8;              // output tiles (n = 8)
    constexpr int CHUNKS = D / 8;          // 16-byte copies in one key's row

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [2][KT][LDS]
    __nv_bfloat16* v_s = k_s + 2 * KT * LDS;                                  // [2][KT][LDS]

    const WorkItem it = items[blockIdx.x];
    if (it.kv_begin >= it.kv_end) {                                           // padding item
        pdl_wait();
        return;
    }
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp / WN, wn = warp % WN;
    const int gid = lane >> 2, tig = lane & 3;

    // the two rows of this thread: gid and gid + 8 of the warp's 16
    int row[2], pos[2], tok[2], hq[2];
    bool live[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        row[i] = it.row0 + wm * 16 + gid + 8 * i;
        live[i] = row[i] < rows_total;
        tok[i] = live[i] ? row[i] / g : 0;
        hq[i] = hk * g + (live[i] ? row[i] % g : 0);
        pos[i] = live[i] ? pos0 + tok[i] : -1;
    }

    pdl_wait();            // q, and the keys and values of this step's tokens, are just written

    // q fragments straight from global memory (read once)
    unsigned qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const __nv_bfloat16* p = q + (size_t)(tok0 + tok[i]) * q_stride + hq[i] * D + kk * 16 +
                                     2 * tig;
            qf[kk][i] = live[i] ? *reinterpret_cast<const unsigned*>(p) : 0u;
            qf[kk][i + 2] = live[i] ? *reinterpret_cast<const unsigned*>(p + 8) : 0u;
        }
    }

    // key range of the tile and of this thread's rows
    const int last_row = min(it.row0 + ROWS, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    int k_lo_true = it.kv_begin;
    if (window > 0) k_lo_true = max(k_lo_true, min_pos - window + 1);
    const int k_lo = (k_lo_true / KT) * KT;
    int lo[2], hi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        lo[i] = it.kv_begin;
        if (window > 0) lo[i] = max(lo[i], pos[i] - window + 1);
        hi[i] = min(it.kv_end, pos[i] + 1);          // pos -1 (dead row): nothing is visible
    }
    // over the warp: is every key of a tile visible to every row?  (rows gid differ per lane)
    int min_hi = min(hi[0], hi[1]), max_lo = max(lo[0], lo[1]);
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        min_hi = min(min_hi, __shfl_xor_sync(0xffffffffu, min_hi, o));
        max_lo = max(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, o));
    }

    const size_t slab = (size_t)page * D;
    auto load_tile = [&](int kt, int stage) {
        __nv_bfloat16* kd = k_s + stage * KT * LDS;
        __nv_bfloat16* vd = v_s + stage * KT * LDS;
        for (int c = threadIdx.x; c < KT * CHUNKS; c += THREADS) {
            const int j = c / CHUNKS, ch = c - j * CHUNKS;
            const int kpos = kt + j;
            bool ok = kpos >= k_lo_true && kpos < k_hi;
            size_t off = 0;
            if (ok) {
                const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
                ok = page_id >= 0 && page_id < num_pages;
                if (ok) off = ((size_t)page_id * kv_heads + hk) * slab + (size_t)(kpos % page) * D +
                              ch * 8;
            }
            cp_async16(kd + j * LDS + ch * 8, k_pages + off, ok);
            cp_async16(vd + j * LDS + ch * 8, v_pages + off, ok);
        }
    };

    float o_acc[DT][4];
#pragma unroll
    for (int j = 0; j < DT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float sl = scale * 1.4426950408889634f;           // scores in the exp2 domain

    load_tile(k_lo, 0);
    cp_async_commit();
    int stage = 0;
    for (int kt = k_lo; kt < k_hi; kt += KT, stage ^= 1) {
        if (kt + KT < k_hi) load_tile(kt + KT, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const __nv_bfloat16* kb = k_s + stage * KT * LDS + wn * NK * LDS;
        const __nv_bfloat16* vb = v_s + stage * KT * LDS + wn * NK * LDS;

        // s = q k^T : 16 rows x NK keys
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                unsigned b[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4(b, kb + ((j + (mat >> 1)) * 8 + r) * LDS + kk * 16 + (mat & 1) * 8);
                mma_bf16(s[j], qf[kk], b[0], b[1]);
                mma_bf16(s[j + 1], qf[kk], b[2], b[3]);
            }
        }

        // masks (only on tiles that reach a limit)
        const int key0 = kt + wn * NK;
        if (key0 + NK > min_hi || key0 < max_lo) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + 2 * tig + (e & 1);
                    const int i = e >> 1;
                    if (key < lo[i] || key >= hi[i]) s[j][e] = -INFINITY;
                }
        }

        // running softmax
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            m_new[0] = fmaxf(m_new[0], fmaxf(s[j][0], s[j][1]));
            m_new[1] = fmaxf(m_new[1], fmaxf(s[j][2], s[j][3]));
        }
        float corr[2], m_use[2], l_add[2] = {0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
            m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
            m_use[i] = m_new[i] == -INFINITY ? 0.0f : m_new[i];
            corr[i] = fast_exp2((m_run[i] - m_use[i]) * sl);        // 0 while m_run is -inf
            m_run[i] = m_new[i];
        }
        unsigned pf[NK / 16][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const float p0 = fast_exp2((s[j][0] - m_use[0]) * sl), p1 = fast_exp2((s[j][1] - m_use[0]) * sl);
            const float p2 = fast_exp2((s[j][2] - m_use[1]) * sl), p3 = fast_exp2((s[j][3] - m_use[1]) * sl);
            l_add[0] += p0 + p1;
            l_add[1] += p2 + p3;
            pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
            pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_add[i];
#pragma unroll
        for (int j = 0; j < DT; ++j) {
            o_acc[j][0] *= corr[0]; o_acc[j][1] *= corr[0];
            o_acc[j][2] *= corr[1]; o_acc[j][3] *= corr[1];
        }

        // o += p v
#pragma unroll
        for (int ks = 0; ks < NK / 16; ++ks) {
#pragma unroll
            for (int jd = 0; jd < DT; jd += 2) {
                unsigned b[4];
                const int mat = lane >> 3, r = lane & 7;
                ldmatrix_x4_trans(b, vb + (ks * 16 + (mat & 1) * 8 + r) * LDS +
                                         (jd + (mat >> 1)) * 8);
                mma_bf16(o_acc[jd], pf[ks], b[0], b[1]);
                mma_bf16(o_acc[jd + 1], pf[ks], b[2], b[3]);
            }
        }
        __syncthreads();                       // this stage may be overwritten by the next load
    }
    cp_async_wait<0>();
    pdl_trigger();

    // row sums live in the 4 lanes of a quad
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }

    if constexpr (WN == 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!live[i]) continue;
            if (it.partial < 0) {
                const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
                __nv_bfloat16* o = out + (size_t)(tok0 + tok[i]) * out_stride + hq[i] * D;
#pragma unroll
                for (int j = 0; j < DT; ++j)
                    *reinterpret_cast<unsigned*>(o + j * 8 + 2 * tig) =
                        pack_bf16(o_acc[j][2 * i] * inv, o_acc[j][2 * i + 1] * inv);
            } else {
                const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + (row[i] - it.row0);
                float* pa = partial_acc + idx * D;
#pragma unroll
                for (int j = 0; j < DT; ++j) {
                    pa[j * 8 + 2 * tig] = o_acc[j][2 * i];
                    pa[j * 8 + 2 * tig + 1] = o_acc[j][2 * i + 1];
                }
                if (tig == 0) {
                    partial_ml[idx * 2] = m_run[i] * scale;      // natural-log domain, as merged
                    partial_ml[idx * 2 + 1] = l_run[i];
                }
            }
        }
    } else {
        // merge the WN warps that split the keys: through shared memory (the tiles are done)
        float* red_o = reinterpret_cast<float*>(smem_raw);             // [WN][16][D]
        float* red_m = red_o + WN * 16 * D;                             // [WN][16]
        float* red_l = red_m + WN * 16;                                 // [WN][16]
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = gid + 8 * i;
            float* dst = red_o + ((size_t)wn * 16 + r) * D;
#pragma unroll
            for (int j = 0; j < DT; ++j) {
                dst[j * 8 + 2 * tig] = o_acc[j][2 * i];
                dst[j * 8 + 2 * tig + 1] = o_acc[j][2 * i + 1];
            }
            if (tig == 0) {
                red_m[wn * 16 + r] = m_run[i];
                red_l[wn * 16 + r] = l_run[i];
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 16 * D; e += THREADS) {
            const int r = e / D, dd = e - r * D;
            const int rr = it.row0 + r;
            if (rr >= rows_total) continue;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < WN; ++w) m = fmaxf(m, red_m[w * 16 + r]);
            float l = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < WN; ++w) {
                const float mw = red_m[w * 16 + r];
                if (mw == -INFINITY) continue;
                const float f = exp2f((mw - m) * sl);
                l += red_l[w * 16 + r] * f;
                acc += red_o[((size_t)w * 16 + r) * D + dd] * f;
            }
            if (it.partial < 0) {
                const int t = rr / g, h = hk * g + rr % g;
                out[(size_t)(tok0 + t) * out_stride + h * D + dd] =
                    __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
            } else {
                const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + r;
                partial_acc[idx * D + dd] = acc;
                if (dd == 0) {
                    partial_ml[idx * 2] = m * scale;
                    partial_ml[idx * 2 + 1] = l;
                }
            }
        }
    }
}

template <int WM, int WN>
int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
           const void* v_pages, const int* block_table, int table_stride, int num_pages,
           const int* seq_slot, const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
           const int* items, int num_items, float* partial_acc, float* partial_ml, int heads,
           int kv_heads, int page, float scale, int window, cudaStream_t s) {
    size_t smem = (size_t)4 * KT * LDS * sizeof(__nv_bfloat16);
    const size_t red = (size_t)WN * 16 * (D + 2) * sizeof(float);
    if (WN > 1 && red > smem) smem = red;
    auto kernel = attn_mma_kernel<WM, WN>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(num_items, kv_heads);
    return de_launch(kernel, grid, dim3(THREADS), smem, s, (const __nv_bfloat16*)q, q_stride,
                     (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages,
                     (const __nv_bfloat16*)v_pages, block_table, table_stride, num_pages, seq_slot,
                     seq_qstart, seq_qlen, seq_pos0, (const WorkItem*)items, partial_acc,
                     partial_ml, heads, kv_heads, page, scale, window);
}

}  // namespace

DE_EXPORT int de_attn_mma_head_dim() { return D; }

// shape 0: wide (64 rows a tile), shape 1: narrow (16 rows a tile)
DE_EXPORT int de_attn_mma(int shape, const void* q, int q_stride, void* out, int out_stride,
                          const void* k_pages, const void* v_pages, const int* block_table,
                          int table_stride, int num_pages, const int* seq_slot,
                          const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                          const int* items, int num_items, float* partial_acc, float* partial_ml,
                          int heads, int kv_heads, int head_dim, int page, float scale, int window,
                          void* stream) {
    if (num_items <= 0) return 0;
    if (head_dim != D || heads % kv_heads != 0) return -2;
    if (q_stride % 2 != 0 || out_stride % 2 != 0) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (shape == 0)
        return launch<4, 1>(q, q_stride, out, out_stride, k_pages, v_pages, block_table,
                            table_stride, num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0, items,
                            num_items, partial_acc, partial_ml, heads, kv_heads, page, scale, window,
                            s);
    return launch<1, 4>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                        num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0, items, num_items,
                        partial_acc, partial_ml, heads, kv_heads, page, scale, window, s);
}

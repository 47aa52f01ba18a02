// Attention over the paged cache, float32 arithmetic on the CUDA cores, for float32 or bfloat16
// storage and any head size up to 256.  It serves the true 32-bit path and every head size that
// the tensor-core kernel does not take.  One kernel does prompt portions and decoded tokens: the
// host cuts the step into work items, each a tile of up to 8 query rows of one sequence and one
// kv head, with a range of keys.
//
// A row is (token, query head within the kv head's group); query head h reads kv head h / g
// (the reference expands k and v with repeat_interleave, src/layers/attention.py:35-36).
// score = (q . k) * scale, scale applied after the product (:38); a key is masked when its
// position is greater than the query's (:41-58) or, with a window, when it is `window` or more
// positions behind; softmax in float32 (:66-69) as a running maximum and sum over tiles of 32
// keys.  Keys come straight from the pages through the block table
// (position -> page, offset: src/distengine/paged_kv_cache.py:165-167); nothing is gathered or
// expanded in memory (the reference copies and expands, paged_kv_cache.py:197-214,318-321).
// A key inside a row's visible range whose page the block table does not hold is masked like a
// key outside the range (never scored as zeros) and recorded in the status word (code 2).
//
// Long key ranges of decoded tokens are cut into chunks that separate blocks work on; each writes
// an unnormalised partial result (accumulator, maximum, sum) into scratch memory, and
// `attn_combine` merges the chunks of a row in ascending order.

#include "common.cuh"

DE_DEFINE_PDL_SWITCH

namespace {

constexpr int ROWS = 8;        // query rows (warps) per block
constexpr int TILE = 32;       // keys per tile: one per lane
constexpr int MAX_D = 256;

struct WorkItem {              // 8 ints, built on the host
    int seq;                   // index into the step's sequence arrays
    int row0;                  // first row of the tile among the sequence's rows of this step
    int kv_begin, kv_end;      // key positions this item covers (before causal / window limits)
    int partial;               // slot in scratch, or -1: write the output directly
    int pad0, pad1, pad2;
};

struct CombineItem {           // 4 ints
    int seq, row0, first_partial, num_partials;
};

template <typename T>
__global__ void __launch_bounds__(ROWS * 32)
attn_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                 const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                 const int* __restrict__ block_table, int table_stride, int num_pages,
                 const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                 const int* __restrict__ seq_qlen, const int* __restrict__ seq_pos0,
                 const WorkItem* __restrict__ items, float* __restrict__ partial_acc,
                 float* __restrict__ partial_ml, int partial_limit, int heads, int kv_heads, int d,
                 int page, float scale, int window, int* __restrict__ status) {
    extern __shared__ float smem[];
    float* Ks = smem;                       // [TILE][d + 1]; column d: 0, or -inf without a page
    float* Vs = Ks + TILE * (d + 1);        // [TILE][d]
    float* Qs = Vs + TILE * d;              // [ROWS][d]

    const WorkItem it = items[blockIdx.x];
    // (an item whose partial slot lies beyond the scratch it was given is skipped like padding)
    if (it.kv_begin >= it.kv_end || it.partial >= partial_limit) {
        pdl_wait();
        return;
    }
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int qlen = seq_qlen[it.seq], pos0 = seq_pos0[it.seq];
    const int slot = seq_slot[it.seq], tok0 = seq_qstart[it.seq];
    const int rows_total = qlen * g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int r = it.row0 + warp;
    const bool active = r < rows_total;
    const int t = active ? r / g : 0;
    const int hq = hk * g + (active ? r % g : 0);
    const int pos = pos0 + t;

    pdl_wait();            // q, and the keys and values of this step's tokens, are just written
    for (int i = lane; i < d; i += 32)
        Qs[warp * d + i] = active ? to_float(q[(size_t)(tok0 + t) * q_stride + hq * d + i]) : 0.0f;

    // key range of the whole tile
    const int last_row = min(it.row0 + ROWS, rows_total) - 1;
    const int max_pos = pos0 + last_row / g, min_pos = pos0 + it.row0 / g;
    const int k_hi = min(it.kv_end, max_pos + 1);
    int k_lo_true = it.kv_begin;
    if (window > 0) k_lo_true = max(k_lo_true, min_pos - window + 1);
    const int k_lo = (k_lo_true / TILE) * TILE;       // tiles sit at absolute positions
    // key range of this warp's row
    int row_lo = it.kv_begin;
    if (window > 0) row_lo = max(row_lo, pos - window + 1);
    const int row_hi = min(it.kv_end, pos + 1);

    float m = -INFINITY, l = 0.0f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.0f;

    const size_t slab = (size_t)page * d;             // one (page, kv head)
    for (int kt = k_lo; kt < k_hi; kt += TILE) {
        __syncthreads();                              // the previous tile has been consumed
        for (int idx = threadIdx.x; idx < TILE * d; idx += ROWS * 32) {
            const int j = idx / d, dd = idx - j * d;
            const int kpos = kt + j;
            float kv = 0.0f, vv = 0.0f;
            bool held = true;
            if (kpos >= k_lo_true && kpos < k_hi) {
                const int page_id = block_table[(size_t)slot * table_stride + kpos / page];
                held = page_id >= 0 && page_id < num_pages;
                if (held) {
                    const size_t off =
                        ((size_t)page_id * kv_heads + hk) * slab + (size_t)(kpos % page) * d + dd;
                    kv = to_float(k_pages[off]);
                    vv = to_float(v_pages[off]);
                }
            }
            Ks[j * (d + 1) + dd] = kv;
            Vs[j * d + dd] = vv;
            if (dd == 0) {
                Ks[j * (d + 1) + d] = held ? 0.0f : -INFINITY;
                if (!held && status != nullptr) atomicExch(status, 2);
            }
        }
        __syncthreads();
        if (!active) continue;

        const int kpos = kt + lane;
        const float* kr = Ks + lane * (d + 1);
        const bool valid = kpos >= row_lo && kpos < row_hi && kr[d] == 0.0f;
        const float* qr = Qs + warp * d;
        float s = 0.0f;
        for (int dd = 0; dd < d; ++dd) s = fmaf(qr[dd], kr[dd], s);
        s = valid ? s * scale : -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;             // nothing of this tile is visible to the row
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);           // 0 when m was -inf
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
        for (int j = 0; j < TILE; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (pj == 0.0f) continue;                 // uniform over the warp
            const float* vr = Vs + j * d;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int dd = lane + 32 * i;
                if (dd < d) acc[i] = fmaf(pj, vr[dd], acc[i]);
            }
        }
        m = m_new;
    }
    pdl_trigger();
    if (!active) return;

    if (it.partial < 0) {
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        T* o = out + (size_t)(tok0 + t) * out_stride + hq * d;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int dd = lane + 32 * i;
            if (dd < d) o[dd] = from_float<T>(acc[i] * inv);
        }
    } else {
        const size_t idx = ((size_t)it.partial * kv_heads + hk) * ROWS + warp;
        float* pa = partial_acc + idx * d;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int dd = lane + 32 * i;
            if (dd < d) pa[dd] = acc[i];
        }
        if (lane == 0) {
            partial_ml[idx * 2] = m;
            partial_ml[idx * 2 + 1] = l;
        }
    }
}

// Merge the chunks of each row, in ascending order of the chunks.
template <typename T>
__global__ void __launch_bounds__(ROWS * 32)
attn_combine_kernel(T* __restrict__ out, int out_stride, const int* __restrict__ seq_qstart,
                    const int* __restrict__ seq_qlen, const CombineItem* __restrict__ items,
                    const float* __restrict__ partial_acc, const float* __restrict__ partial_ml,
                    int partial_limit, int heads, int kv_heads, int d, int rows_per_tile) {
    const CombineItem it = items[blockIdx.x];
    pdl_wait();
    pdl_trigger();
    if (it.num_partials <= 0) return;
    // slots beyond the scratch that was given: nothing is read, the rows are left as they are
    if (it.first_partial < 0 || it.first_partial > partial_limit - it.num_partials) return;
    const int hk = blockIdx.y;
    const int g = heads / kv_heads;
    const int rows_total = seq_qlen[it.seq] * g;
    const int lane = threadIdx.x & 31;
    for (int w = threadIdx.x >> 5; w < rows_per_tile; w += ROWS) {
        const int r = it.row0 + w;
        if (r >= rows_total) continue;
        const int t = r / g, hq = hk * g + r % g;
        float m = -INFINITY;
        for (int c = 0; c < it.num_partials; ++c) {
            const size_t idx = ((size_t)(it.first_partial + c) * kv_heads + hk) * rows_per_tile + w;
            m = fmaxf(m, partial_ml[idx * 2]);
        }
        float l = 0.0f;
        float acc[MAX_D / 32];
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.0f;
        for (int c = 0; c < it.num_partials; ++c) {
            const size_t idx = ((size_t)(it.first_partial + c) * kv_heads + hk) * rows_per_tile + w;
            const float mc = partial_ml[idx * 2];
            if (mc == -INFINITY) continue;            // the chunk held no visible key
            const float f = expf(mc - m);
            l += partial_ml[idx * 2 + 1] * f;
            const float* pa = partial_acc + idx * d;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int dd = lane + 32 * i;
                if (dd < d) acc[i] = fmaf(pa[dd], f, acc[i]);
            }
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        T* o = out + (size_t)(seq_qstart[it.seq] + t) * out_stride + hq * d;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int dd = lane + 32 * i;
            if (dd < d) o[dd] = from_float<T>(acc[i] * inv);
        }
    }
}

}  // namespace

DE_EXPORT int de_attn_simt_rows_per_tile() { return ROWS; }

static int launch_simt(int dtype, const void* q, int q_stride, void* out, int out_stride,
                       const void* k_pages, const void* v_pages, const int* block_table,
                       int table_stride, int num_pages, const int* seq_slot,
                       const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                       const int* items, int num_items, float* partial_acc, float* partial_ml,
                       int partial_limit, int heads, int kv_heads, int d, int page, float scale,
                       int window, int* status, void* stream);
static int launch_combine(int dtype, void* out, int out_stride, const int* seq_qstart,
                          const int* seq_qlen, const int* items, int num_items,
                          const float* partial_acc, const float* partial_ml, int partial_limit,
                          int heads, int kv_heads, int d, int rows_per_tile, void* stream);

DE_EXPORT int de_attn_simt(int dtype, const void* q, int q_stride, void* out, int out_stride,
                           const void* k_pages, const void* v_pages, const int* block_table,
                           int table_stride, int num_pages, const int* seq_slot,
                           const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                           const int* items, int num_items, float* partial_acc, float* partial_ml,
                           int heads, int kv_heads, int d, int page, float scale, int window,
                           int* status, void* stream) {
    return launch_simt(dtype, q, q_stride, out, out_stride, k_pages, v_pages, block_table,
                       table_stride, num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0, items,
                       num_items, partial_acc, partial_ml, 0x7fffffff, heads, kv_heads, d, page,
                       scale, window, status, stream);
}

// `partial_limit`: partial slots that the scratch holds (work items that name a slot beyond it are
// skipped); `status`: may be null.
static int launch_simt(int dtype, const void* q, int q_stride, void* out, int out_stride,
                       const void* k_pages, const void* v_pages, const int* block_table,
                       int table_stride, int num_pages, const int* seq_slot,
                       const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
                       const int* items, int num_items, float* partial_acc, float* partial_ml,
                       int partial_limit, int heads, int kv_heads, int d, int page, float scale,
                       int window, int* status, void* stream) {
    if (num_items <= 0) return 0;
    if (d <= 0 || d > MAX_D || heads % kv_heads != 0) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(TILE * (d + 1) + TILE * d + ROWS * d) * sizeof(float);
    dim3 grid(num_items, kv_heads);
    cudaError_t e;
#define LAUNCH(T)                                                                               \
    do {                                                                                        \
        if (smem > 48 * 1024) {                                                                 \
            e = cudaFuncSetAttribute(attn_simt_kernel<T>,                                       \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
            if (e != cudaSuccess) return (int)e;                                                \
        }                                                                                       \
        return de_launch(attn_simt_kernel<T>, grid, dim3(ROWS * 32), smem, s, (const T*)q,      \
                         q_stride, (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages,   \
                         block_table, table_stride, num_pages, seq_slot, seq_qstart, seq_qlen,  \
                         seq_pos0, (const WorkItem*)items, partial_acc, partial_ml,             \
                         partial_limit, heads, kv_heads, d, page, scale, window, status);       \
    } while (0)
    if (dtype == DE_BF16) LAUNCH(__nv_bfloat16);
    LAUNCH(float);
#undef LAUNCH
}

// `rows_per_tile`: rows of a tile in the partial layout (8 for the kernel above; the tensor-core
// kernel writes the same layout with its own tile height).
DE_EXPORT int de_attn_combine(int dtype, void* out, int out_stride, const int* seq_qstart,
                              const int* seq_qlen, const int* items, int num_items,
                              const float* partial_acc, const float* partial_ml, int heads,
                              int kv_heads, int d, int rows_per_tile, void* stream) {
    return launch_combine(dtype, out, out_stride, seq_qstart, seq_qlen, items, num_items,
                          partial_acc, partial_ml, 0x7fffffff, heads, kv_heads, d, rows_per_tile,
                          stream);
}

static int launch_combine(int dtype, void* out, int out_stride, const int* seq_qstart,
                          const int* seq_qlen, const int* items, int num_items,
                          const float* partial_acc, const float* partial_ml, int partial_limit,
                          int heads, int kv_heads, int d, int rows_per_tile, void* stream) {
    if (num_items <= 0) return 0;
    if (d <= 0 || d > MAX_D) return -2;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(num_items, kv_heads);
    if (dtype == DE_BF16)
        return de_launch(attn_combine_kernel<__nv_bfloat16>, grid, dim3(ROWS * 32), 0, s,
                         (__nv_bfloat16*)out, out_stride, seq_qstart, seq_qlen,
                         (const CombineItem*)items, partial_acc, partial_ml, partial_limit, heads,
                         kv_heads, d, rows_per_tile);
    return de_launch(attn_combine_kernel<float>, grid, dim3(ROWS * 32), 0, s, (float*)out,
                     out_stride, seq_qstart, seq_qlen, (const CombineItem*)items, partial_acc,
                     partial_ml, partial_limit, heads, kv_heads, d, rows_per_tile);
}

// ------------------------------------------------------------------------------------------
// The variant that allocates nothing: see attention_static_scratch.h for who needs it and the
// rules.  The scratch for the partial results is this file-scope device array.  Its name is a
// device symbol: host code must not pass it to a kernel as if it were a pointer (on the host the
// name stands for a shadow object, not for device memory); the device address is looked up once
// per device with cudaGetSymbolAddress and that pointer is what the kernels get.
// ------------------------------------------------------------------------------------------
#include <cstdio>
#include <mutex>

#include "attention_static_scratch.h"

static __device__ __align__(256) float g_static_scratch[DE_ATTN_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {};       // per device, filled at the first call there
std::mutex g_scratch_mutex;
thread_local char g_static_error[256] = "";

// The device address of the array on the current device; looked up at the first call on it.
int static_scratch_address(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MAX_DEVICES) return -11;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_address[device] = static_cast<float*>(p);
    }
    *address = g_scratch_address[device];
    return 0;
}
}  // namespace

DE_EXPORT const char* de_attn_static_scratch_error(void) { return g_static_error; }

DE_EXPORT int de_attn_simt_static_scratch(
    int dtype, const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
    const void* v_pages, const int* block_table, int table_stride, int num_pages,
    const int* seq_slot, const int* seq_qstart, const int* seq_qlen, const int* seq_pos0,
    const int* items, int num_items, const int* combine_items, int num_combine, int num_partials,
    int heads, int kv_heads, int head_dim, int page, float scale, int window, void* stream) {
    g_static_error[0] = '\0';
    if (num_items <= 0) return 0;
    if (head_dim <= 0 || head_dim > MAX_D || kv_heads <= 0 || heads % kv_heads != 0 ||
        num_partials < 0) {
        std::snprintf(g_static_error, sizeof(g_static_error),
                      "de_attn_simt_static_scratch: head_dim %d (1..%d), heads %d, kv_heads %d or "
                      "num_partials %d cannot be used", head_dim, MAX_D, heads, kv_heads,
                      num_partials);
        return -2;
    }
    const long long rows = (long long)num_partials * kv_heads * ROWS;
    const long long need = rows * (head_dim + 2);
    if (need > DE_ATTN_STATIC_SCRATCH_FLOATS) {
        std::snprintf(g_static_error, sizeof(g_static_error),
                      "de_attn_simt_static_scratch: %d partial results x %d kv heads x %d rows x "
                      "(head_dim %d + 2) = %lld floats, the built-in scratch array holds %d; use "
                      "de_attn_simt with scratch of your own, or fewer chunks",
                      num_partials, kv_heads, ROWS, head_dim, need, DE_ATTN_STATIC_SCRATCH_FLOATS);
        return DE_ATTN_STATIC_TOO_LARGE;
    }
    float* scratch = nullptr;
    const int status = static_scratch_address(&scratch);
    if (status != 0) {
        std::snprintf(g_static_error, sizeof(g_static_error),
                      "de_attn_simt_static_scratch: the scratch array's device address could not "
                      "be looked up (code %d)", status);
        return status;
    }
    float* partial_acc = scratch;                               // [rows][head_dim]
    float* partial_ml = scratch + rows * head_dim;              // [rows][2]
    // the kernels are told how many partial slots the array holds for this call: an item that
    // names a slot at or beyond num_partials writes and merges nothing
    int code = launch_simt(dtype, q, q_stride, out, out_stride, k_pages, v_pages, block_table,
                           table_stride, num_pages, seq_slot, seq_qstart, seq_qlen, seq_pos0,
                           items, num_items, partial_acc, partial_ml, num_partials, heads,
                           kv_heads, head_dim, page, scale, window, nullptr, stream);
    if (code != 0) return code;
    return launch_combine(dtype, out, out_stride, seq_qstart, seq_qlen, combine_items,
                          num_combine, partial_acc, partial_ml, num_partials, heads, kv_heads,
                          head_dim, ROWS, stream);
}

// Differential attention over a paged cache: two score maps a head, one set of values.
//
// A layer of this kind projects its input to queries [heads, 2, dim], keys [kv_heads, 2, dim] and
// values [kv_heads, vdim]; query head h reads key/value head h / (heads / kv_heads). Each of the two
// maps is a softmax attention of its own over the same values, a1 and a2, and a head's result is
//     o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * post_scale,   o <- o * sigmoid(gate)
// with one lambda for the layer. Before the maps, queries, keys and values pass a short causal
// convolution over time on each channel (y_t = sum_j w[c, j] u_(t - taps + 1 + j), zeros before the
// sequence's start); the last taps - 1 projected rows of a sequence are kept as state. Queries and
// keys are then divided by their root mean square over dim, per head and map, and multiplied by a
// weight of dim entries. Key j is visible from position i when j <= i and (window == 0 or
// i - j < window or j < keep_first): a sliding window that also keeps a sequence's first tokens.
//
// Cache rows: keys [pages, kv_heads, page_size, 2 * dim] (the two maps side by side) and values
// [pages, kv_heads, page_size, vdim]; every page of a sequence is kept, the window is a mask.
//
// Kernels here:
//  * prepare: convolution, norms, the query rows and the cache write, a warp per (row, map or value
//    head); with one token a sequence it also moves the convolution's state on;
//  * state: the convolution's state after a step of several tokens;
//  * attention, general: any element type and width up to 256; a block per (row, head), keys dealt
//    to its four warps by position only, so a row's result does not depend on the batch or on how
//    the sequence was cut into steps;
//  * attention on the tensor cores (bfloat16): see the second half of this file.
// Convolution sums, norm sums, scores, softmax, the weighted sums and everything after them are
// 32-bit.
#include "common.cuh"

#ifndef KIDI_DIFF_DIM
#define KIDI_DIFF_DIM 0        // the maps' width the tensor-core kernels are compiled for (0: none)
#endif
#ifndef KIDI_DIFF_VDIM
#define KIDI_DIFF_VDIM 0
#endif

constexpr int MAX_TAPS = 32;

struct DiffGeometry {
    const int* table;      // [slots + 1, pages_per_seq]
    int pages_per_seq;
    int page_shift;
    int heads, kv_heads, dim, vdim;
};

struct DiffTables {
    const int* row_seq;    // [rows] (-1: padding row)
    const int* row_pos;
    const int* seq_slot;
    const int* seq_start;
    const int* seq_len;
    const int* seq_row0;
};

__device__ __forceinline__ long long diff_page_row(const DiffGeometry& g, int slot, int position, int kv_head) {
    const int page = g.table[(long long)slot * g.pages_per_seq + (position >> g.page_shift)];
    const int within = position & ((1 << g.page_shift) - 1);
    return (((long long)page * g.kv_heads + kv_head) << g.page_shift) + within;
}

struct DiffPrepareArgs {
    const void* proj;      // [rows, ld]: q maps, k maps, v heads (then whatever else the projection makes)
    long long ld;
    const void* conv;      // [channels, taps] or null (no convolution)
    int taps;
    void* state;           // [slots + 1, taps - 1, channels]
    const void* q_norm;    // [dim]
    const void* k_norm;
    void* q_out;           // [rows, heads * 2 * dim]
    void* k_cache;
    void* v_cache;
    DiffGeometry geometry;
    DiffTables tables;
    int rows, seqs;
    float eps;
    int move_state;        // 1: one token a sequence, the state is moved on here
};

// V consecutive elements of a row, as floats (V = 2: a bfloat16 pair in one 4-byte access).
template <typename T, int V> __device__ __forceinline__ void load_elements(const T* p, float (&out)[V]) {
#pragma unroll
    for (int v = 0; v < V; ++v) out[v] = to_float(p[v]);
}
template <> __device__ __forceinline__ void load_elements<bf16, 2>(const bf16* p, float (&out)[2]) {
    const float2 pair = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    out[0] = pair.x;
    out[1] = pair.y;
}
template <typename T, int V> __device__ __forceinline__ void store_elements(T* p, const float (&in)[V]) {
#pragma unroll
    for (int v = 0; v < V; ++v) p[v] = from_float<T>(in[v]);
}
template <> __device__ __forceinline__ void store_elements<bf16, 2>(bf16* p, const float (&in)[2]) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(in[0], in[1]);
}

// One warp per (row, unit): units are the 2 * heads query maps, the 2 * kv_heads key maps and the
// kv_heads value heads, in the projection's order. A lane takes V consecutive channels at a time
// (V = 2 for bfloat16 rows of even widths: 128 bytes a warp and access).
template <typename T, typename TW, int V>
__global__ void __launch_bounds__(128) diff_prepare_kernel(DiffPrepareArgs a) {
    constexpr int ROUNDS = 8 / V;
    const DiffGeometry& g = a.geometry;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_units = 2 * g.heads, k_units = 2 * g.kv_heads, units = q_units + k_units + g.kv_heads;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)a.rows * units) return;
    const int row = (int)(item / units), unit = (int)(item - (long long)row * units);
    const int seq = a.tables.row_seq[row];
    if (seq < 0) return;
    const int position = a.tables.row_pos[row], start = a.tables.seq_start[seq], row0 = a.tables.seq_row0[seq];
    const int slot = a.tables.seq_slot[seq];
    const int channels = (q_units + k_units) * g.dim + g.kv_heads * g.vdim;
    int base, width;
    if (unit < q_units + k_units) { base = unit * g.dim; width = g.dim; }
    else { base = (q_units + k_units) * g.dim + (unit - q_units - k_units) * g.vdim; width = g.vdim; }
    const T* proj = (const T*)a.proj;
    const TW* conv = (const TW*)a.conv;
    const int taps = conv ? a.taps : 1;
    T* state = (T*)a.state + (long long)slot * (taps - 1) * channels;

    float values[ROUNDS][V];
    float square = 0.f;
#pragma unroll
    for (int i = 0; i < ROUNDS; ++i) {
        const int c = (lane + 32 * i) * V;
        float y[V];
#pragma unroll
        for (int v = 0; v < V; ++v) y[v] = 0.f;
        if (c < width) {
            const int channel = base + c;
            if (!conv) {
                load_elements<T, V>(proj + (long long)row * a.ld + channel, y);
            } else {
                for (int j = 0; j < taps; ++j) {
                    const int t = position - (taps - 1) + j;
                    float u[V];
#pragma unroll
                    for (int v = 0; v < V; ++v) u[v] = 0.f;
                    if (t >= start) load_elements<T, V>(proj + (long long)(row0 + t - start) * a.ld + channel, u);
                    else if (t >= 0) load_elements<T, V>(state + (long long)(t - (start - (taps - 1))) * channels + channel, u);
#pragma unroll
                    for (int v = 0; v < V; ++v) y[v] = fmaf(to_float(conv[(long long)(channel + v) * taps + j]), u[v], y[v]);
                    // One token a sequence: this lane alone reads and writes its channels' state, and row j - 1
                    // was read an iteration ago.
                    if (a.move_state && j > 0) store_elements<T, V>(state + (long long)(j - 1) * channels + channel, u);
                }
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            values[i][v] = y[v];
            square = fmaf(y[v], y[v], square);
        }
    }
    if (unit < q_units + k_units) {
        const TW* weight = (const TW*)(unit < q_units ? a.q_norm : a.k_norm);
        const float inv = 1.0f / sqrtf(warp_sum(square) / (float)g.dim + a.eps);
        T* out;
        if (unit < q_units) {
            out = (T*)a.q_out + (long long)row * q_units * g.dim + (long long)unit * g.dim;
        } else {
            const int k_unit = unit - q_units;
            out = (T*)a.k_cache + diff_page_row(g, slot, position, k_unit >> 1) * (2 * g.dim) + (k_unit & 1) * g.dim;
        }
#pragma unroll
        for (int i = 0; i < ROUNDS; ++i) {
            const int c = (lane + 32 * i) * V;
            if (c < width) {
                float normed[V];
#pragma unroll
                for (int v = 0; v < V; ++v) normed[v] = values[i][v] * inv * to_float(weight[c + v]);
                store_elements<T, V>(out + c, normed);
            }
        }
    } else {
        T* out = (T*)a.v_cache + diff_page_row(g, slot, position, unit - q_units - k_units) * g.vdim;
#pragma unroll
        for (int i = 0; i < ROUNDS; ++i) {
            const int c = (lane + 32 * i) * V;
            if (c < width) store_elements<T, V>(out + c, values[i]);
        }
    }
}

// The state after a step: the projected rows of the sequence's last taps - 1 positions. A thread
// owns a (sequence, channel) and walks the state's rows upwards: row i takes what row i + len held
// (or a row of the step), which no earlier iteration has overwritten.
template <typename T>
__global__ void diff_state_kernel(DiffPrepareArgs a, int channels) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (long long)a.seqs * channels) return;
    const int seq = (int)(index / channels), channel = (int)(index - (long long)seq * channels);
    const int slot = a.tables.seq_slot[seq], start = a.tables.seq_start[seq], len = a.tables.seq_len[seq];
    const int row0 = a.tables.seq_row0[seq];
    if (a.tables.row_seq[row0] < 0) return;
    const int keep = a.taps - 1;
    T* state = (T*)a.state + (long long)slot * keep * channels;
    const T* proj = (const T*)a.proj;
    for (int i = 0; i < keep; ++i) {
        const int t = start + len - keep + i;
        T value = from_float<T>(0.f);
        if (t >= start) value = proj[(long long)(row0 + t - start) * a.ld + channel];
        else if (t >= 0) value = state[(long long)(t - (start - keep)) * channels + channel];
        state[(long long)i * channels + channel] = value;
    }
}

KIDI_API int kidi_diff_prepare(const DiffPrepareArgs* args, int dtype, int weight_dtype, cudaStream_t stream) {
    const DiffPrepareArgs& a = *args;
    const DiffGeometry& g = a.geometry;
    if (a.rows <= 0) return 0;
    if (g.dim <= 0 || g.dim > 256 || g.vdim <= 0 || g.vdim > 256 || g.heads % g.kv_heads) return KIDI_REFUSED_SIZE;
    if (a.conv && (a.taps < 1 || a.taps > MAX_TAPS)) return KIDI_REFUSED_SIZE;
    const long long items = (long long)a.rows * (2 * g.heads + 3 * g.kv_heads);
    const unsigned blocks = (unsigned)((items + 3) / 4);
    int status;
    // bfloat16 rows of even widths: a lane takes pairs
    const bool pairs = dtype == KIDI_BF16 && !(g.dim & 1) && !(g.vdim & 1) && !(a.ld & 1) && !((uintptr_t)a.proj & 3) &&
                       !((uintptr_t)a.state & 3) && !((uintptr_t)a.q_out & 3) && !((uintptr_t)a.k_cache & 3) &&
                       !((uintptr_t)a.v_cache & 3);
#define KIDI_CASE(D, T, W, TW, V)                                                                  \
    if (dtype == D && weight_dtype == W && pairs == (V == 2)) {                                    \
        status = kidi_launch(diff_prepare_kernel<T, TW, V>, blocks, 128, 0, stream, a);           \
        if (status || !a.conv || a.taps < 2 || a.move_state) return status;                       \
        const int channels = 2 * (g.heads + g.kv_heads) * g.dim + g.kv_heads * g.vdim;            \
        const long long total = (long long)a.seqs * channels;                                     \
        return kidi_launch(diff_state_kernel<T>, (unsigned)((total + 255) / 256), 256, 0, stream, a, channels); \
    }
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float, 1)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16, 1)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, 1)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, 1)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, 2)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, 2)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
struct DiffAttentionArgs {
    const void* q;         // [rows, heads * 2 * dim]
    const void* gate;      // [rows, ldg]: head h at h * vdim; null: no gate
    long long ldg;
    const void* k_cache;
    const void* v_cache;
    DiffGeometry geometry;
    DiffTables tables;
    void* out;             // [rows, heads * vdim]
    int rows, seqs, max_new;
    int window;            // 0: every earlier key is visible
    int keep_first;
    float scale, lambda, post_scale, eps;
    float* partial;        // workspace of the split form
    int splits;
};

// What follows the two maps, for one head of one row: `o1`, `o2` are a lane's entries lane, lane + 32,
// ... of the two weighted sums (already divided by their softmax sums).
template <typename T>
__device__ __forceinline__ void diff_finish(const DiffAttentionArgs& a, int row, int head, int lane, const float* o1,
                                            const float* o2) {
    const int e = a.geometry.vdim;
    float o[8], square = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        o[i] = lane + 32 * i < e ? o1[i] - a.lambda * o2[i] : 0.f;
        square = fmaf(o[i], o[i], square);
    }
    const float inv = 1.0f / sqrtf(warp_sum(square) / (float)e + a.eps) * a.post_scale;
    T* out = (T*)a.out + (long long)row * a.geometry.heads * e + (long long)head * e;
    const T* gate = a.gate ? (const T*)a.gate + (long long)row * a.ldg + (long long)head * e : nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c < e) {
            float value = o[i] * inv;
            if (gate) value *= 1.0f / (1.0f + expf(-to_float(gate[c])));
            out[c] = from_float<T>(value);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) diff_attention_generic_kernel(DiffAttentionArgs a) {
    __shared__ float query[2][256];
    __shared__ float part_acc[4][2][256];
    __shared__ float part_max[4][2], part_sum[4][2];
    const DiffGeometry& g = a.geometry;
    const int row = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = g.dim, e = g.vdim;
    const int seq = a.tables.row_seq[row];
    if (seq < 0) {
        T* out = (T*)a.out + (long long)row * g.heads * e + (long long)head * e;
        for (int c = threadIdx.x; c < e; c += 128) out[c] = from_float<T>(0.f);
        return;
    }
    const int position = a.tables.row_pos[row], slot = a.tables.seq_slot[seq];
    const int first = a.window > 0 ? max(0, position - a.window + 1) : 0;
    const int kept = min(a.keep_first, first);          // first tokens that the window no longer covers
    const int count = kept + position - first + 1;
    const int kv_head = head / (g.heads / g.kv_heads);
    const T* q = (const T*)a.q + ((long long)row * g.heads + head) * 2 * d;
    for (int c = threadIdx.x; c < 2 * d; c += 128) query[c >= d][c >= d ? c - d : c] = to_float(q[c]);
    __syncthreads();

    float best[2] = {-INFINITY, -INFINITY}, denom[2] = {0.f, 0.f};
    float acc[2][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[0][i] = acc[1][i] = 0.f;
    for (int n = warp; n < count; n += 4) {
        const int u = n < kept ? n : first + (n - kept);
        const long long at = diff_page_row(g, slot, u, kv_head);
        const T* key = (const T*)a.k_cache + at * (2 * d);
        const T* value = (const T*)a.v_cache + at * e;
        float dot[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < d) {
                dot[0] = fmaf(query[0][c], to_float(key[c]), dot[0]);
                dot[1] = fmaf(query[1][c], to_float(key[d + c]), dot[1]);
            }
        }
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = lane + 32 * i < e ? to_float(value[lane + 32 * i]) : 0.f;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const float score = warp_sum(dot[m]) * a.scale;
            const float next = fmaxf(best[m], score);
            const float keep = expf(best[m] - next), weight = expf(score - next);
            denom[m] = denom[m] * keep + weight;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[m][i] = acc[m][i] * keep + weight * v[i];
            best[m] = next;
        }
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        if (lane == 0) { part_max[warp][m] = best[m]; part_sum[warp][m] = denom[m]; }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (lane + 32 * i < e) part_acc[warp][m][lane + 32 * i] = acc[m][i];
    }
    __syncthreads();
    if (warp) return;
    float o[2][8];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float top = part_max[0][m];
#pragma unroll
        for (int w = 1; w < 4; ++w) top = fmaxf(top, part_max[w][m]);
        float total = 0.f, factor[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            factor[w] = part_max[w][m] == -INFINITY ? 0.f : expf(part_max[w][m] - top);
            total += part_sum[w][m] * factor[w];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            float value = 0.f;
            if (c < e)
#pragma unroll
                for (int w = 0; w < 4; ++w) value += part_acc[w][m][c] * factor[w];
            o[m][i] = value / total;
        }
    }
    diff_finish<T>(a, row, head, lane, o[0], o[1]);
}

KIDI_API int kidi_diff_attention_generic(const DiffAttentionArgs* args, int dtype, cudaStream_t stream) {
    const DiffAttentionArgs& a = *args;
    const DiffGeometry& g = a.geometry;
    if (a.rows <= 0) return 0;
    if (g.dim <= 0 || g.dim > 256 || g.vdim <= 0 || g.vdim > 256 || g.heads % g.kv_heads || g.heads > 65535)
        return KIDI_REFUSED_SIZE;
    dim3 grid(a.rows, g.heads);
    if (dtype == KIDI_F32) return kidi_launch(diff_attention_generic_kernel<float>, grid, 128, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(diff_attention_generic_kernel<bf16>, grid, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
// The tensor-core kernels (bfloat16), compiled for one pair of widths.
//
// A block takes rows of one sequence that share a key/value head. In a prompt: 64 rows = 64 / (heads per
// key/value head) consecutive tokens times those heads, and eight warps: a warp takes 16 rows, all 64
// keys of a tile and ONE of the two maps (so that a map's weighted sum of 16 rows by vdim columns is what
// a warp holds, and twice as many warps fit a multiprocessor as with both maps to a warp); the warps of
// the second map hand their result to those of the first through shared memory at the end. With one
// token a sequence: four warps, the 16 (or fewer) heads of the token, each warp both maps and a
// quarter of a tile's keys, merged through shared memory at the end. A tile is a 64-token page of
// the cache (keys of both maps, values), copied with cp.async into one of two buffers while the
// other is used. The tiles a block visits are the pages of its window and, before them, the pages
// of the kept first tokens. Per map: S = Q K^T (mma.sync m16n8k16, fragments through ldmatrix), the
// mask, an online softmax in 32-bit, P in bfloat16, O += P V. The two maps' sums stay in registers;
// their difference, its norm and the gate are applied there too. With `splits` > 1 (one token a
// sequence, long windows) the tiles of a (sequence, key/value head) are dealt to several blocks
// whose results meet in a workspace and a second kernel.
#if KIDI_DIFF_DIM > 0
namespace tensor {

constexpr int DIM = KIDI_DIFF_DIM, VDIM = KIDI_DIFF_VDIM;
constexpr int KS = 2 * DIM + 8;      // elements between rows of a key or query tile in shared memory
constexpr int VS = VDIM + 8;
constexpr int TILE = 64;
constexpr int NV = VDIM / 8;         // output column tiles
constexpr int STAGE = VDIM + 4;      // floats between rows of the merge stage
static_assert(DIM % 16 == 0 && VDIM % 16 == 0 && DIM <= 128 && VDIM <= 128, "widths the kernel takes");

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t address = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
    const uint32_t address = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void copy16(bf16* shared, const bf16* global) {
    const uint32_t address = (uint32_t)__cvta_generic_to_shared(shared);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(address), "l"(global));
}
__device__ __forceinline__ uint32_t pack2(float low, float high) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
}
__device__ __forceinline__ float exp2_fast(float v) {        // 2^v; 0 for -inf
    float result;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(result) : "f"(v));
    return result;
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// ROW_WARPS 4: prompts (64 rows a block); 1: one token a sequence (16 rows, the warps share a tile's keys).
template <int ROW_WARPS>
__global__ void __launch_bounds__(ROW_WARPS == 4 ? 256 : 128, 2) diff_attention_tensor_kernel(DiffAttentionArgs a) {
    constexpr int MAPS = ROW_WARPS == 4 ? 1 : 2;          // maps a warp takes
    constexpr int THREADS = ROW_WARPS == 4 ? 256 : 128;
    constexpr int KEY_WARPS = 4 / ROW_WARPS;
    constexpr int ROWS = 16 * ROW_WARPS;
    constexpr int KEYS_W = TILE / KEY_WARPS;
    constexpr int NT = KEYS_W / 8;
    extern __shared__ __align__(16) unsigned char shared_bytes[];
    bf16* q_s = reinterpret_cast<bf16*>(shared_bytes);
    bf16* k_s = q_s + ROWS * KS;
    bf16* v_s = k_s + 2 * TILE * KS;

    const DiffGeometry& g = a.geometry;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = g.heads / g.kv_heads;
    const int seq = blockIdx.y, kv_head = blockIdx.z % g.kv_heads, split = blockIdx.z / g.kv_heads;
    const int tokens = ROW_WARPS == 4 ? ROWS / group : 1;
    const int len = a.tables.seq_len[seq], start = a.tables.seq_start[seq], row0 = a.tables.seq_row0[seq];
    // the blocks with the most keys to walk (a sequence's last tokens) start first
    const int t0 = (gridDim.x - 1 - blockIdx.x) * tokens;
    if (t0 >= len) return;
    const int live_tokens = min(tokens, len - t0), live_rows = live_tokens * group;
    bf16* out = (bf16*)a.out;
    if (a.tables.row_seq[row0] < 0) {          // a padding sequence of a captured step: zeros, nothing read
        if (split == 0 && a.splits == 1)
            for (int i = tid; i < live_rows * VDIM; i += THREADS) {
                const int r = i / VDIM, c = i - r * VDIM;
                out[((long long)(row0 + t0 + r / group) * g.heads + kv_head * group + r % group) * VDIM + c] =
                    __float2bfloat16_rn(0.f);
            }
        return;
    }
    const int slot = a.tables.seq_slot[seq];
    const int p_low = start + t0, p_high = start + t0 + live_tokens - 1;
    const int low_page = a.window > 0 ? max(0, p_low - a.window + 1) >> 6 : 0;
    const int high_page = p_high >> 6;
    const int kept_tiles = min((a.keep_first + TILE - 1) >> 6, low_page);
    const int tiles = kept_tiles + high_page - low_page + 1;
    const int share = (tiles + a.splits - 1) / a.splits;
    const int first_tile = split * share, end_tile = min(tiles, first_tile + share);

    const bf16* k_cache = (const bf16*)a.k_cache;
    const bf16* v_cache = (const bf16*)a.v_cache;
    const int* table = g.table + (long long)slot * g.pages_per_seq;
    auto page_of = [&](int tile) { return tile < kept_tiles ? tile : low_page + tile - kept_tiles; };
    // A tile's page id is read from the block table an iteration before the tile is asked for, so that the
    // copies of the next tile do not wait for that read.
    auto load_tile = [&](int page_id, int buffer) {
        const long long at = ((long long)page_id * g.kv_heads + kv_head) << 6;
        const bf16* keys = k_cache + at * (2 * DIM);
        const bf16* values = v_cache + at * VDIM;
        bf16* k_to = k_s + buffer * TILE * KS;
        bf16* v_to = v_s + buffer * TILE * VS;
        for (int i = tid; i < TILE * (2 * DIM / 8); i += THREADS) {
            const int r = i / (2 * DIM / 8), piece = i - r * (2 * DIM / 8);
            copy16(k_to + r * KS + piece * 8, keys + r * (2 * DIM) + piece * 8);
        }
        for (int i = tid; i < TILE * (VDIM / 8); i += THREADS) {
            const int r = i / (VDIM / 8), piece = i - r * (VDIM / 8);
            copy16(v_to + r * VS + piece * 8, values + r * VDIM + piece * 8);
        }
        asm volatile("cp.async.commit_group;");
    };

    // prompts: warps 0..3 take the first map of rows 16 w.., warps 4..7 the second; one token: each warp both maps
    const int own_map = MAPS == 1 ? warp >> 2 : 0;
    const int row_warp = MAPS == 1 ? warp & 3 : 0, key0 = MAPS == 1 ? 0 : warp * KEYS_W;
    const int row_a = row_warp * 16 + (lane >> 2), row_b = row_a + 8;
    // A row's position; -1 for rows beyond the block's live rows: they see nothing.
    const int pos_a = row_a < live_rows ? start + t0 + row_a / group : -1;
    const int pos_b = row_b < live_rows ? start + t0 + row_b / group : -1;
    const float scale_log2 = a.scale * 1.4426950408889634f;

    float o[MAPS][NV][4];
    float top_a[MAPS], top_b[MAPS], sum_a[MAPS], sum_b[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
        top_a[m] = top_b[m] = -INFINITY;
        sum_a[m] = sum_b[m] = 0.f;
#pragma unroll
        for (int n = 0; n < NV; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[m][n][e] = 0.f;
    }

    if (first_tile < end_tile) load_tile(table[page_of(first_tile)], 0);
    int next_page_id = first_tile + 1 < end_tile ? table[page_of(first_tile + 1)] : 0;
    // The block's query rows (while the first tile is on its way): row r is token t0 + r / group, head
    // kv_head * group + r % group.
    const bf16* q = (const bf16*)a.q;
    for (int i = tid; i < ROWS * (2 * DIM / 8); i += THREADS) {
        const int r = i / (2 * DIM / 8), piece = i - r * (2 * DIM / 8);
        uint4 value = make_uint4(0u, 0u, 0u, 0u);
        if (r < live_rows)
            value = *reinterpret_cast<const uint4*>(
                q + ((long long)(row0 + t0 + r / group) * g.heads + kv_head * group + r % group) * (2 * DIM) + piece * 8);
        *reinterpret_cast<uint4*>(q_s + r * KS + piece * 8) = value;
    }
    for (int tile = first_tile; tile < end_tile; ++tile) {
        const int buffer = (tile - first_tile) & 1;
        if (tile + 1 < end_tile) {
            load_tile(next_page_id, buffer ^ 1);
            if (tile + 2 < end_tile) next_page_id = table[page_of(tile + 2)];
            asm volatile("cp.async.wait_group 1;");
        } else {
            asm volatile("cp.async.wait_group 0;");
        }
        __syncthreads();
        const bf16* k_tile = k_s + buffer * TILE * KS;
        const bf16* v_tile = v_s + buffer * TILE * VS;
        const int tile_key = page_of(tile) << 6, key_base = tile_key + key0;
        // A tile that every row of the block sees whole needs no mask (most tiles of a long sequence).
        const bool whole = tile_key + TILE - 1 <= p_low &&
                           (a.window <= 0 || p_high - tile_key < a.window || tile_key + TILE - 1 < a.keep_first);
#pragma unroll
        for (int m = 0; m < MAPS; ++m) {
            const int map = MAPS == 1 ? own_map : m;          // which of the two maps of queries and keys
            float s[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DIM / 16; ++ks) {
                uint32_t qa[4];
                ldmatrix_x4(qa, q_s + (row_warp * 16 + (lane & 15)) * KS + map * DIM + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int n2 = 0; n2 < NT / 2; ++n2) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, k_tile + (key0 + n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + map * DIM + ks * 16 +
                                        ((lane >> 3) & 1) * 8);
                    mma_bf16(s[2 * n2], qa, kb[0], kb[1]);
                    mma_bf16(s[2 * n2 + 1], qa, kb[2], kb[3]);
                }
            }
            // Scores stay unscaled; the scale (times log2 e) enters the exponent's multiply-add.
            float most_a = -INFINITY, most_b = -INFINITY;
            if (!whole) {
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int u = key_base + n * 8 + (lane & 3) * 2 + (e & 1);
                        const int p = e < 2 ? pos_a : pos_b;
                        const bool seen = u <= p && (a.window <= 0 || p - u < a.window || u < a.keep_first);
                        if (!seen) s[n][e] = -INFINITY;
                    }
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                most_a = fmaxf(most_a, fmaxf(s[n][0], s[n][1]));
                most_b = fmaxf(most_b, fmaxf(s[n][2], s[n][3]));
            }
            const float next_a = fmaxf(top_a[m], quad_max(most_a)), next_b = fmaxf(top_b[m], quad_max(most_b));
            const float base_a = next_a == -INFINITY ? 0.f : next_a * scale_log2;
            const float base_b = next_b == -INFINITY ? 0.f : next_b * scale_log2;
            const float keep_a = exp2_fast(top_a[m] * scale_log2 - base_a), keep_b = exp2_fast(top_b[m] * scale_log2 - base_b);
            top_a[m] = next_a;
            top_b[m] = next_b;
            float add_a = 0.f, add_b = 0.f;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                s[n][0] = exp2_fast(fmaf(s[n][0], scale_log2, -base_a)); s[n][1] = exp2_fast(fmaf(s[n][1], scale_log2, -base_a));
                s[n][2] = exp2_fast(fmaf(s[n][2], scale_log2, -base_b)); s[n][3] = exp2_fast(fmaf(s[n][3], scale_log2, -base_b));
                add_a += s[n][0] + s[n][1];
                add_b += s[n][2] + s[n][3];
            }
            sum_a[m] = sum_a[m] * keep_a + add_a;
            sum_b[m] = sum_b[m] * keep_b + add_b;
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                o[m][n][0] *= keep_a; o[m][n][1] *= keep_a;
                o[m][n][2] *= keep_b; o[m][n][3] *= keep_b;
            }
#pragma unroll
            for (int kk = 0; kk < KEYS_W / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack2(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack2(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < NV / 2; ++n2) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, v_tile + (key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + n2 * 16 +
                                              (lane >> 4) * 8);
                    mma_bf16(o[m][2 * n2], pa, vb[0], vb[1]);
                    mma_bf16(o[m][2 * n2 + 1], pa, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
        sum_a[m] = quad_sum(sum_a[m]);
        sum_b[m] = quad_sum(sum_b[m]);
        top_a[m] *= scale_log2;           // from here on the largest scores are exponents of two (-inf stays)
        top_b[m] *= scale_log2;
    }

    if constexpr (KEY_WARPS > 1) {
        // The four warps hold the same 16 rows over different keys: they meet in shared memory, behind the
        // query rows, and the first warp adds them up.
        float* stage = reinterpret_cast<float*>(shared_bytes + ((ROWS * KS * 2 + 15) & ~15));   // [4][2][16][STAGE]
        float* stats = stage + 4 * 2 * 16 * STAGE;                                               // [4][2][16][2]
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float* mine = stage + ((warp * 2 + m) * 16) * STAGE;
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                const int c = n * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(mine + (lane >> 2) * STAGE + c) = make_float2(o[m][n][0], o[m][n][1]);
                *reinterpret_cast<float2*>(mine + ((lane >> 2) + 8) * STAGE + c) = make_float2(o[m][n][2], o[m][n][3]);
            }
            if ((lane & 3) == 0) {
                float* at = stats + ((warp * 2 + m) * 16) * 2;
                at[(lane >> 2) * 2] = top_a[m]; at[(lane >> 2) * 2 + 1] = sum_a[m];
                at[((lane >> 2) + 8) * 2] = top_b[m]; at[((lane >> 2) + 8) * 2 + 1] = sum_b[m];
            }
        }
        __syncthreads();
        if (warp) return;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float best_a = -INFINITY, best_b = -INFINITY;
            for (int w = 0; w < 4; ++w) {
                const float* at = stats + ((w * 2 + m) * 16) * 2;
                best_a = fmaxf(best_a, at[(lane >> 2) * 2]);
                best_b = fmaxf(best_b, at[((lane >> 2) + 8) * 2]);
            }
            float total_a = 0.f, total_b = 0.f;
#pragma unroll
            for (int n = 0; n < NV; ++n) o[m][n][0] = o[m][n][1] = o[m][n][2] = o[m][n][3] = 0.f;
            for (int w = 0; w < 4; ++w) {
                const float* at = stats + ((w * 2 + m) * 16) * 2;
                const float has_a = at[(lane >> 2) * 2], has_b = at[((lane >> 2) + 8) * 2];
                const float factor_a = has_a == -INFINITY ? 0.f : exp2f(has_a - best_a);
                const float factor_b = has_b == -INFINITY ? 0.f : exp2f(has_b - best_b);
                total_a += at[(lane >> 2) * 2 + 1] * factor_a;
                total_b += at[((lane >> 2) + 8) * 2 + 1] * factor_b;
                const float* theirs = stage + ((w * 2 + m) * 16) * STAGE;
#pragma unroll
                for (int n = 0; n < NV; ++n) {
                    const int c = n * 8 + (lane & 3) * 2;
                    const float2 upper = *reinterpret_cast<const float2*>(theirs + (lane >> 2) * STAGE + c);
                    const float2 lower = *reinterpret_cast<const float2*>(theirs + ((lane >> 2) + 8) * STAGE + c);
                    o[m][n][0] += upper.x * factor_a; o[m][n][1] += upper.y * factor_a;
                    o[m][n][2] += lower.x * factor_b; o[m][n][3] += lower.y * factor_b;
                }
            }
            top_a[m] = best_a; top_b[m] = best_b;
            sum_a[m] = total_a; sum_b[m] = total_b;
        }
    }

    // Each map's weighted sum divided by its softmax sum (a row without a key, which only a share of
    // the tiles can be, gives zeros and a zero sum).
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
        const float inv_a = sum_a[m] > 0.f ? 1.0f / sum_a[m] : 0.f, inv_b = sum_b[m] > 0.f ? 1.0f / sum_b[m] : 0.f;
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            o[m][n][0] *= inv_a; o[m][n][1] *= inv_a;
            o[m][n][2] *= inv_b; o[m][n][3] *= inv_b;
        }
    }
    // The second map's result, where the first map's is: in the same warp (one token a sequence), or handed over
    // by the warp four further on through shared memory (prompts), behind the query rows.
    float second[NV][4];
    if constexpr (MAPS == 2) {
#pragma unroll
        for (int n = 0; n < NV; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) second[n][e] = o[1][n][e];
    } else {
        float* stage = reinterpret_cast<float*>(shared_bytes + ((ROWS * KS * 2 + 15) & ~15)) + row_warp * 16 * STAGE;
        __syncthreads();
        if (own_map == 1) {
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                const int c = n * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(stage + (lane >> 2) * STAGE + c) = make_float2(o[0][n][0], o[0][n][1]);
                *reinterpret_cast<float2*>(stage + ((lane >> 2) + 8) * STAGE + c) = make_float2(o[0][n][2], o[0][n][3]);
            }
        }
        __syncthreads();
        if (own_map == 1) return;
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int c = n * 8 + (lane & 3) * 2;
            const float2 upper = *reinterpret_cast<const float2*>(stage + (lane >> 2) * STAGE + c);
            const float2 lower = *reinterpret_cast<const float2*>(stage + ((lane >> 2) + 8) * STAGE + c);
            second[n][0] = upper.x; second[n][1] = upper.y;
            second[n][2] = lower.x; second[n][3] = lower.y;
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? row_b : row_a;
        const bool live = r < live_rows;
        const long long row = row0 + t0 + (live ? r / group : 0);
        const int head = kv_head * group + (live ? r % group : 0);
        if constexpr (MAPS == 2) {
            if (a.splits > 1) {
                if (live) {
                    float* to = a.partial + ((row * g.heads + head) * a.splits + split) * (2 * VDIM + 4);
#pragma unroll
                    for (int n = 0; n < NV; ++n) {
                        *reinterpret_cast<float2*>(to + n * 8 + (lane & 3) * 2) = make_float2(o[0][n][2 * half], o[0][n][2 * half + 1]);
                        *reinterpret_cast<float2*>(to + VDIM + n * 8 + (lane & 3) * 2) =
                            make_float2(second[n][2 * half], second[n][2 * half + 1]);
                    }
                    if ((lane & 3) == 0) {
                        to[2 * VDIM] = half ? top_b[0] : top_a[0]; to[2 * VDIM + 1] = half ? sum_b[0] : sum_a[0];
                        to[2 * VDIM + 2] = half ? top_b[MAPS - 1] : top_a[MAPS - 1];
                        to[2 * VDIM + 3] = half ? sum_b[MAPS - 1] : sum_a[MAPS - 1];
                    }
                }
                continue;
            }
        }
        float square = 0.f;
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const float x = o[0][n][2 * half] - a.lambda * second[n][2 * half];
            const float y = o[0][n][2 * half + 1] - a.lambda * second[n][2 * half + 1];
            o[0][n][2 * half] = x;
            o[0][n][2 * half + 1] = y;
            square = fmaf(x, x, fmaf(y, y, square));
        }
        const float inv = 1.0f / sqrtf(quad_sum(square) / (float)VDIM + a.eps) * a.post_scale;
        if (!live) continue;
        bf16* to = out + (row * g.heads + head) * VDIM;
        const bf16* gate = a.gate ? (const bf16*)a.gate + row * a.ldg + (long long)head * VDIM : nullptr;
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int c = n * 8 + (lane & 3) * 2;
            float x = o[0][n][2 * half] * inv, y = o[0][n][2 * half + 1] * inv;
            if (gate) {
                const float2 opened = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + c));
                x *= 1.0f / (1.0f + expf(-opened.x));
                y *= 1.0f / (1.0f + expf(-opened.y));
            }
            *reinterpret_cast<__nv_bfloat162*>(to + c) = __floats2bfloat162_rn(x, y);
        }
    }
}

// The shares of a (row, head) meet: a warp a (row, head).
__global__ void __launch_bounds__(128) diff_combine_kernel(DiffAttentionArgs a) {
    const DiffGeometry& g = a.geometry;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)a.rows * g.heads) return;
    const int row = (int)(item / g.heads), head = (int)(item - (long long)row * g.heads);
    if (a.tables.row_seq[row] < 0) {
        bf16* out = (bf16*)a.out + ((long long)row * g.heads + head) * VDIM;
        for (int c = lane; c < VDIM; c += 32) out[c] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* from = a.partial + item * a.splits * (2 * VDIM + 4);
    float o[2][8];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float best = -INFINITY;
        for (int s = 0; s < a.splits; ++s) best = fmaxf(best, from[s * (2 * VDIM + 4) + 2 * VDIM + 2 * m]);
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[m][i] = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float* share = from + s * (2 * VDIM + 4);
            const float has = share[2 * VDIM + 2 * m], sum = share[2 * VDIM + 2 * m + 1];
            const float factor = (has == -INFINITY || sum <= 0.f) ? 0.f : sum * exp2f(has - best);
            total += factor;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (lane + 32 * i < VDIM) o[m][i] += share[m * VDIM + lane + 32 * i] * factor;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) o[m][i] /= total;
    }
    diff_finish<bf16>(a, row, head, lane, o[0], o[1]);
}

}  // namespace tensor

KIDI_API int kidi_diff_attention_tensor(const DiffAttentionArgs* args, cudaStream_t stream) {
    using namespace tensor;
    const DiffAttentionArgs& a = *args;
    const DiffGeometry& g = a.geometry;
    if (a.rows <= 0) return 0;
    if (g.dim != DIM || g.vdim != VDIM || g.page_shift != 6 || g.heads % g.kv_heads || a.splits < 1) return KIDI_REFUSED_SIZE;
    const int group = g.heads / g.kv_heads;
    const bool one_token = a.max_new == 1;
    if (group > (one_token ? 16 : 64) || a.seqs > 65535 || (long long)g.kv_heads * a.splits > 65535) return KIDI_REFUSED_SIZE;
    if (a.splits > 1 && (!one_token || !a.partial)) return KIDI_REFUSED_SIZE;
    const size_t tiles = (size_t)(2 * TILE * KS + 2 * TILE * VS) * sizeof(bf16);
    int status;
    if (one_token) {
        const size_t rows = ((size_t)16 * KS * sizeof(bf16) + 15) & ~(size_t)15;
        const size_t stage = (size_t)(4 * 2 * 16 * STAGE + 4 * 2 * 16 * 2) * sizeof(float);
        const size_t shared = rows + (tiles > stage ? tiles : stage);
        static bool set = false;
        if (!set) {
            cudaError_t error = cudaFuncSetAttribute(diff_attention_tensor_kernel<1>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
            if (error != cudaSuccess) return (int)error;
            set = true;
        }
        status = kidi_launch(diff_attention_tensor_kernel<1>, dim3(1, a.seqs, g.kv_heads * a.splits), 128, shared, stream, a);
        if (status || a.splits == 1) return status;
        const long long items = (long long)a.rows * g.heads;
        return kidi_launch(diff_combine_kernel, (unsigned)((items + 3) / 4), 128, 0, stream, a);
    }
    const size_t handed = (size_t)4 * 16 * STAGE * sizeof(float);          // the second map's results on their way
    const size_t shared = (((size_t)64 * KS * sizeof(bf16) + 15) & ~(size_t)15) + (tiles > handed ? tiles : handed);
    static bool set = false;
    if (!set) {
        cudaError_t error = cudaFuncSetAttribute(diff_attention_tensor_kernel<4>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (error != cudaSuccess) return (int)error;
        set = true;
    }
    const int tokens = 64 / group;
    return kidi_launch(diff_attention_tensor_kernel<4>, dim3((a.max_new + tokens - 1) / tokens, a.seqs, g.kv_heads), 256,
                       shared, stream, a);
}
#endif

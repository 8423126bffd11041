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

constexpr int MAX_TAPS = 8;

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

// One warp per (row, unit): units are the 2 * heads query maps, the 2 * kv_heads key maps and the
// kv_heads value heads, in the projection's order.
template <typename T, typename TW>
__global__ void __launch_bounds__(128) diff_prepare_kernel(DiffPrepareArgs a) {
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

    float values[8];
    float square = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        float y = 0.f;
        if (c < width) {
            const int channel = base + c;
            if (!conv) {
                y = to_float(proj[(long long)row * a.ld + channel]);
            } else {
                for (int j = 0; j < taps; ++j) {
                    const int t = position - (taps - 1) + j;
                    float u = 0.f;
                    if (t >= start) u = to_float(proj[(long long)(row0 + t - start) * a.ld + channel]);
                    else if (t >= 0) u = to_float(state[(long long)(t - (start - (taps - 1))) * channels + channel]);
                    y = fmaf(to_float(conv[(long long)channel * taps + j]), u, y);
                    // One token a sequence: this lane alone reads and writes its channel's state, and row j - 1
                    // was read an iteration ago.
                    if (a.move_state && j > 0) state[(long long)(j - 1) * channels + channel] = from_float<T>(u);
                }
            }
        }
        values[i] = y;
        square = fmaf(y, y, square);
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
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < width) out[c] = from_float<T>(values[i] * inv * to_float(weight[c]));
        }
    } else {
        T* out = (T*)a.v_cache + diff_page_row(g, slot, position, unit - q_units - k_units) * g.vdim;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = lane + 32 * i;
            if (c < width) out[c] = from_float<T>(values[i]);
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
#define KIDI_CASE(D, T, W, TW)                                                                     \
    if (dtype == D && weight_dtype == W) {                                                         \
        status = kidi_launch(diff_prepare_kernel<T, TW>, blocks, 128, 0, stream, a);              \
        if (status || !a.conv || a.taps < 2 || a.move_state) return status;                       \
        const int channels = 2 * (g.heads + g.kv_heads) * g.dim + g.kv_heads * g.vdim;            \
        const long long total = (long long)a.seqs * channels;                                     \
        return kidi_launch(diff_state_kernel<T>, (unsigned)((total + 255) / 256), 256, 0, stream, a, channels); \
    }
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16)
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

// Attention over a cached latent: what a token leaves in the cache is one row [c | k_rot] per layer, c the
// normalised latent (rank values) from which every head's keys and values are linear maps, k_rot a rotated key part
// (rot_dim values) that all heads share. With the key map folded into the query (q_lat = W_uk^T q, per head) a head's
// score against token u is (q_lat . c_u + q_rot . k_rot_u) * scale and its result is the weighted sum of the c_u,
// to which the value map is applied afterwards: one key/value "head" of width rank + rot_dim whose values are the
// first rank entries of its keys.
//
// Two kernels for any element type: `latent_prepare` (RMS norm of the latent, interleaved rotation of the shared key
// part and of the queries' rotated parts, cache write) and `latent_attention` (causal softmax attention of every row
// over its sequence's cached rows). Norm sums, angles, scores, softmax and the weighted sums are 32-bit. The order
// of a row's additions depends on its position only.
#include "common.cuh"

struct LatentPrepareArgs {
    const void* q;          // [rows, ldq]: per head [dim plain | rot_dim to rotate]
    long long ldq;
    void* folded;           // [rows, ldf]: per head [rank (filled by the caller) | rot_dim rotated, written here]
    long long ldf;
    void* kv;               // [rows, ldkv]: [rank latent | rot_dim shared key part], or null (nothing is cached)
    long long ldkv;
    int write_back;         // the normalised latent and the rotated key part also replace the row of kv
    int skip_queries;       // only the cache entries are made
    const float* kv_norm;   // [rank]
    const float* cos_table; // [positions, rotary_dims / 2]
    const float* sin_table;
    const int* row_seq;     // [rows] (-1: padding row, skipped)
    const int* row_pos;
    const int* seq_slot;
    void* cache;            // storage of this schedule entry [pages, 1, page, rank + rot_dim]
    CacheGeometry geometry;
    int rows, heads, dim, rot_dim, rotary_dims, rank;
    float eps;
};

// One warp per (row, unit): units 0..heads-1 are the query heads, unit `heads` is the row's cache entry.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(LatentPrepareArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.skip_queries ? 0 : a.heads;
    const int units = heads + (a.kv ? 1 : 0);
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)a.rows * units) return;
    const int row = (int)(item / units), unit = (int)(item - (long long)row * units);
    const int seq = a.row_seq[row];
    if (seq < 0) return;
    const int position = a.row_pos[row];
    const int half = a.rotary_dims / 2;
    const float* cosine = a.cos_table + (long long)position * half;
    const float* sine = a.sin_table + (long long)position * half;
    const T* source;
    T* target;
    T* second = nullptr;    // the row of kv, when it is written back
    if (unit < heads) {
        source = (const T*)a.q + row * a.ldq + (long long)unit * (a.dim + a.rot_dim) + a.dim;
        target = (T*)a.folded + row * a.ldf + (long long)unit * (a.rank + a.rot_dim) + a.rank;
    } else {
        T* latent = (T*)a.kv + row * a.ldkv;
        T* cached = (T*)a.cache + cache_row_offset(a.geometry, a.seq_slot[seq], position, 0);
        float square = 0.f;
        for (int c = lane; c < a.rank; c += 32) {
            const float value = to_float(latent[c]);
            square = fmaf(value, value, square);
        }
        const float inv = 1.0f / sqrtf(warp_sum(square) / (float)a.rank + a.eps);
        for (int c = lane; c < a.rank; c += 32) {
            const T normed = from_float<T>(to_float(latent[c]) * inv * a.kv_norm[c]);
            cached[c] = normed;
            if (a.write_back) latent[c] = normed;
        }
        source = latent + a.rank;
        target = cached + a.rank;
        if (a.write_back) second = latent + a.rank;
    }
    // entries 2i and 2i+1 turn by the angle of pair i; entries from rotary_dims on pass unchanged
    for (int i = lane; i < half; i += 32) {
        const float u = to_float(source[2 * i]), v = to_float(source[2 * i + 1]);
        const float c = cosine[i], s = sine[i];
        const T first = from_float<T>(u * c - v * s), other = from_float<T>(v * c + u * s);
        target[2 * i] = first;
        target[2 * i + 1] = other;
        if (second) { second[2 * i] = first; second[2 * i + 1] = other; }   // the lane's own pair: read above
    }
    for (int c = a.rotary_dims + lane; c < a.rot_dim; c += 32) target[c] = source[c];
}

KIDI_API int kidi_latent_prepare(const LatentPrepareArgs* args, int dtype, cudaStream_t stream) {
    const LatentPrepareArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.skip_queries && !a.kv) return 0;
    if (a.heads <= 0 || a.dim < 0 || a.rot_dim < 0 || a.rank <= 0 || a.rotary_dims < 0 || (a.rotary_dims & 1) ||
        a.rotary_dims > a.rot_dim)
        return KIDI_REFUSED_SIZE;
    const long long items = (long long)a.rows * ((a.skip_queries ? 0 : a.heads) + (a.kv ? 1 : 0));
    if ((items + 3) / 4 > 0x7fffffffLL) return KIDI_REFUSED_SIZE;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (dtype == KIDI_F32) return kidi_launch(latent_prepare_kernel<float>, blocks, 128, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(latent_prepare_kernel<bf16>, blocks, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
struct LatentAttentionArgs {
    const void* folded;     // [rows, ldf]: per head [q_lat (rank) | q_rot (rot_dim)]
    long long ldf;
    const void* cache;      // [pages, 1, page, rank + rot_dim]
    CacheGeometry geometry;
    void* out;              // [rows, ldo]: per head the weighted sum of the latents (rank values)
    long long ldo;
    const int* row_seq;     // [rows] (-1: padding row: output zeros)
    const int* row_pos;
    const int* seq_slot;
    int rows, heads, rank, rot_dim, window;   // window 0: every earlier token is visible
    float scale;
};

// One block of 4 warps per (row, head). Warp w takes tokens first+w, first+w+4, ... in ascending order with an
// online softmax; the four partial results are merged in warp order. CHUNKS * 32 >= rank + rot_dim.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(128) latent_attention_kernel(LatentAttentionArgs a) {
    __shared__ float query[CHUNKS * 32];
    __shared__ float part_acc[4][CHUNKS * 32];
    __shared__ float part_max[4], part_sum[4];
    const int row = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int width = a.rank + a.rot_dim;
    T* out = (T*)a.out + row * a.ldo + (long long)head * a.rank;
    const int seq = a.row_seq[row];
    if (seq < 0) {
        for (int c = threadIdx.x; c < a.rank; c += 128) out[c] = from_float<T>(0.f);
        return;
    }
    const int position = a.row_pos[row];
    const int first = a.window > 0 ? max(0, position - a.window + 1) : 0;
    const int slot = a.seq_slot[seq];
    const T* q = (const T*)a.folded + row * a.ldf + (long long)head * width;
    for (int c = threadIdx.x; c < CHUNKS * 32; c += 128) query[c] = c < width ? to_float(q[c]) : 0.f;
    __syncthreads();

    float best = -INFINITY, denom = 0.f;
    float acc[CHUNKS];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) acc[i] = 0.f;
    for (int u = first + warp; u <= position; u += 4) {
        const T* entry = (const T*)a.cache + cache_row_offset(a.geometry, slot, u, 0);
        float kept[CHUNKS];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) {
            const int c = lane + 32 * i;
            kept[i] = c < width ? to_float(entry[c]) : 0.f;
            dot = fmaf(query[c], kept[i], dot);       // both are zero beyond `width`
        }
        const float score = warp_sum(dot) * a.scale;
        const float next = fmaxf(best, score);
        const float keep = expf(best - next);  // 0 on the first token (best = -inf)
        const float weight = expf(score - next);
        denom = denom * keep + weight;
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) acc[i] = acc[i] * keep + weight * kept[i];
        best = next;
    }
    if (lane == 0) { part_max[warp] = best; part_sum[warp] = denom; }
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) part_acc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float top = part_max[0];
#pragma unroll
    for (int w = 1; w < 4; ++w) top = fmaxf(top, part_max[w]);
    float total = 0.f, factor[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        factor[w] = part_max[w] == -INFINITY ? 0.f : expf(part_max[w] - top);
        total += part_sum[w] * factor[w];
    }
    for (int c = threadIdx.x; c < a.rank; c += 128) {
        float value = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) value += part_acc[w][c] * factor[w];
        out[c] = from_float<T>(value / total);
    }
}

template <typename T>
static int launch_latent_attention(const LatentAttentionArgs& a, cudaStream_t stream) {
    const int width = a.rank + a.rot_dim;
    dim3 grid(a.rows, a.heads);
    if (width <= 128) return kidi_launch(latent_attention_kernel<T, 4>, grid, 128, 0, stream, a);
    if (width <= 256) return kidi_launch(latent_attention_kernel<T, 8>, grid, 128, 0, stream, a);
    if (width <= 384) return kidi_launch(latent_attention_kernel<T, 12>, grid, 128, 0, stream, a);
    if (width <= 640) return kidi_launch(latent_attention_kernel<T, 20>, grid, 128, 0, stream, a);
    return KIDI_REFUSED_SIZE;
}

KIDI_API int kidi_latent_attention(const LatentAttentionArgs* args, int dtype, cudaStream_t stream) {
    const LatentAttentionArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.heads <= 0 || a.heads > 65535 || a.rank <= 0 || a.rot_dim < 0) return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32) return launch_latent_attention<float>(a, stream);
    if (dtype == KIDI_BF16) return launch_latent_attention<bf16>(a, stream);
    return KIDI_REFUSED_DTYPE;
}

// ---------------------------------------------------------------------------
// The unfolded form for prompts: every head's keys and values are computed from the latents of the step's rows
// and packed, with the queries, into the matrix [rows, 3 * heads * D] (D = dim + rot_dim) that the prompt
// attention kernels of grouped-query attention take: heads of [q_plain | q_rot turned], then heads of
// [k_plain | shared rotated key part], then heads of [value | zeros up to D].
struct LatentPackArgs {
    const void* q;          // [rows, ldq]: per head [dim | rot_dim not yet turned]
    long long ldq;
    const void* latent;     // [rows, ldl]: [rank normalised | rot_dim turned] (as the cache holds them)
    long long ldl;
    const void* unfolded;   // [rows, ldu]: heads*dim plain keys, then heads*vdim values
    long long ldu;
    void* packed;           // [rows, ldp]
    long long ldp;
    const float* cos_table;
    const float* sin_table;
    const int* row_seq;
    const int* row_pos;
    int rows, heads, dim, rot_dim, rotary_dims, rank, vdim;
};

template <typename T>
__global__ void __launch_bounds__(128) latent_pack_kernel(LatentPackArgs a) {
    const int row = blockIdx.x;
    const int D = a.dim + a.rot_dim, half = a.rotary_dims / 2;
    const int position = a.row_seq[row] < 0 ? 0 : a.row_pos[row];
    const float* cosine = a.cos_table + (long long)position * half;
    const float* sine = a.sin_table + (long long)position * half;
    const T* q = (const T*)a.q + row * a.ldq;
    const T* latent = (const T*)a.latent + row * a.ldl;
    const T* unfolded = (const T*)a.unfolded + row * a.ldu;
    T* packed = (T*)a.packed + row * a.ldp;
    const int per_section = a.heads * D;
    for (int index = threadIdx.x; index < 3 * per_section; index += 128) {
        const int section = index / per_section, within = index - section * per_section;
        const int head = within / D, c = within - head * D;
        T value;
        if (section == 0) {
            const T* source = q + head * D;
            if (c < a.dim || c >= a.dim + a.rotary_dims) {
                value = source[c];
            } else {
                const int j = c - a.dim, i = j >> 1;
                const float u = to_float(source[a.dim + 2 * i]), v = to_float(source[a.dim + 2 * i + 1]);
                value = from_float<T>((j & 1) ? v * cosine[i] + u * sine[i] : u * cosine[i] - v * sine[i]);
            }
        } else if (section == 1) {
            value = c < a.dim ? unfolded[head * a.dim + c] : latent[a.rank + c - a.dim];
        } else {
            value = c < a.vdim ? unfolded[a.heads * a.dim + head * a.vdim + c] : from_float<T>(0.f);
        }
        packed[index] = value;
    }
}

KIDI_API int kidi_latent_pack(const LatentPackArgs* args, int dtype, cudaStream_t stream) {
    const LatentPackArgs& a = *args;
    if (a.rows <= 0) return 0;
    if (a.heads <= 0 || a.vdim > a.dim + a.rot_dim || a.rotary_dims > a.rot_dim || (a.rotary_dims & 1)) return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32) return kidi_launch(latent_pack_kernel<float>, a.rows, 128, 0, stream, a);
    if (dtype == KIDI_BF16) return kidi_launch(latent_pack_kernel<bf16>, a.rows, 128, 0, stream, a);
    return KIDI_REFUSED_DTYPE;
}

// Rows of the step as the cache holds them: out[r] = the cached entry of row r's sequence at row r's position
// (for a layer that reads another layer's cached rows). Padding rows get zeros.
template <typename T>
__global__ void __launch_bounds__(128)
latent_gather_kernel(const T* __restrict__ cache, CacheGeometry geometry, T* __restrict__ out, long long ldo,
                     const int* __restrict__ row_seq, const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                     int width) {
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    T* target = out + row * ldo;
    if (seq < 0) {
        for (int c = threadIdx.x; c < width; c += 128) target[c] = from_float<T>(0.f);
        return;
    }
    const T* entry = cache + cache_row_offset(geometry, seq_slot[seq], row_pos[row], 0);
    for (int c = threadIdx.x; c < width; c += 128) target[c] = entry[c];
}

KIDI_API int kidi_latent_gather(const void* cache, const CacheGeometry* geometry, void* out, long long ldo,
                                const int* row_seq, const int* row_pos, const int* seq_slot, int rows, int width,
                                int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == KIDI_F32)
        return kidi_launch(latent_gather_kernel<float>, rows, 128, 0, stream, (const float*)cache, *geometry,
                           (float*)out, ldo, row_seq, row_pos, seq_slot, width);
    if (dtype == KIDI_BF16)
        return kidi_launch(latent_gather_kernel<bf16>, rows, 128, 0, stream, (const bf16*)cache, *geometry, (bf16*)out,
                           ldo, row_seq, row_pos, seq_slot, width);
    return KIDI_REFUSED_DTYPE;
}

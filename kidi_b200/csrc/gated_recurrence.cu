// A gated linear recurrence per head whose write strength is the complement of its forget gate (HGRN2):
//     q_t = silu(q~_t)                                  [dim]
//     f_t = l + (1 - l) * sigmoid(f~_t + b)             [dim]   l: a lower bound per channel
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T         [dim, vdim]
//     o_t = S_t^T q_t   (then divided by its root mean square over vdim, times a weight shared by the heads)
// q~, f~, v are the columns of one fused projection [q~ | f~ | v]. The state S lives in 32-bit floats per cache
// slot and is carried from token to token; gates, state, read-out and the norm are 32-bit.
//
// The recurrence is elementwise in S, so the columns v of a head's state are independent: a block takes 32
// columns of one (sequence, head) and walks the sequence's rows of the step in order. Warp g of its eight owns the
// state rows d = g R .. g R + R - 1 of those columns in registers (R = ceil(dim / 8)); the gates and queries of 16
// tokens at a time are computed once a block into shared memory; the eight partial read-outs of a column meet in
// shared memory and are added in the order of g. A token's result therefore depends on the sizes only: not on
// what else is in the step, nor on how the sequence was cut into steps. The read-out leaves the kernel
// unnormalised (its columns lie in different blocks); the norm over vdim is a kernel of its own.
#include "common.cuh"

struct GatedRecurrenceArgs {
    const void* qfv;       // [rows, ld]: heads*dim of q~, heads*dim of f~, heads*vdim of v
    long long ld;
    const float* f_bias;   // [heads*dim]
    const float* lower;    // [heads*dim]
    float* state;          // [slots + 1, heads, dim, vdim]
    void* out;             // [rows, ldo]: heads*vdim, the unnormalised read-out
    long long ldo;
    const int* row_seq;    // [rows] (-1: padding)
    const int* seq_slot;   // [seqs]
    const int* seq_row0;   // [seqs]
    const int* seq_len;    // [seqs]
    int seqs, heads, dim, vdim;
};

namespace {
constexpr int GROUPS = 8;       // warps of a block: each owns a slice of the state's rows
constexpr int COLUMNS = 32;     // state columns of a block: one a lane
constexpr int CHUNK = 16;       // tokens whose gates are staged at a time

template <typename T, int R>
__global__ void __launch_bounds__(GROUPS * COLUMNS) gated_recurrence_kernel(GatedRecurrenceArgs a) {
    extern __shared__ float shared[];
    const int seq = blockIdx.x, head = blockIdx.y;
    const int row0 = a.seq_row0[seq], count = a.seq_len[seq];
    if (count <= 0 || a.row_seq[row0] < 0) return;       // a padding sequence touches no state
    const int dim = a.dim, vdim = a.vdim;
    constexpr int PADDED = GROUPS * R;                   // dim rounded up: rows beyond dim hold q = 0, f = 1
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int v = blockIdx.z * COLUMNS + lane;
    const bool live = v < vdim;
    float* qs = shared;                                  // [CHUNK][PADDED]
    float* fs = qs + CHUNK * PADDED;                     // [CHUNK][PADDED]
    float* vs = fs + CHUNK * PADDED;                     // [CHUNK][COLUMNS]
    float* partial = vs + CHUNK * COLUMNS;               // [CHUNK][GROUPS][COLUMNS]
    float* state = a.state + ((long long)a.seq_slot[seq] * a.heads + head) * dim * vdim;
    float S[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int d = g * R + j;
        S[j] = live && d < dim ? state[(long long)d * vdim + v] : 0.f;
    }
    const float* bias = a.f_bias + head * dim;
    const float* lower = a.lower + head * dim;
    for (int t0 = 0; t0 < count; t0 += CHUNK) {
        const int tokens = min(CHUNK, count - t0);
        for (int index = threadIdx.x; index < tokens * PADDED; index += GROUPS * COLUMNS) {
            const int t = index / PADDED, d = index - t * PADDED;
            float q = 0.f, f = 1.f;
            if (d < dim) {
                const T* row = (const T*)a.qfv + (long long)(row0 + t0 + t) * a.ld;
                const float raw = to_float(row[head * dim + d]);
                q = raw / (1.0f + expf(-raw));
                const float gate = 1.0f / (1.0f + expf(-(to_float(row[(a.heads + head) * dim + d]) + bias[d])));
                f = lower[d] + (1.0f - lower[d]) * gate;
            }
            qs[index] = q;
            fs[index] = f;
        }
        for (int index = threadIdx.x; index < tokens * COLUMNS; index += GROUPS * COLUMNS) {
            const int t = index / COLUMNS, c = index - t * COLUMNS;
            const int column = blockIdx.z * COLUMNS + c;
            const T* row = (const T*)a.qfv + (long long)(row0 + t0 + t) * a.ld;
            vs[index] = column < vdim ? to_float(row[2 * a.heads * dim + head * vdim + column]) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < tokens; ++t) {
            const float value = vs[t * COLUMNS + lane];
            const float* q = qs + t * PADDED + g * R;    // the same addresses for a whole warp: broadcasts
            const float* f = fs + t * PADDED + g * R;
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const float s = f[j] * S[j] + (1.0f - f[j]) * value;
                S[j] = s;
                sum = fmaf(s, q[j], sum);
            }
            partial[(t * GROUPS + g) * COLUMNS + lane] = sum;
        }
        __syncthreads();
        for (int index = threadIdx.x; index < tokens * COLUMNS; index += GROUPS * COLUMNS) {
            const int t = index / COLUMNS, c = index - t * COLUMNS;
            const int column = blockIdx.z * COLUMNS + c;
            if (column >= vdim) continue;
            float total = 0.f;
#pragma unroll
            for (int k = 0; k < GROUPS; ++k) total += partial[(t * GROUPS + k) * COLUMNS + c];
            ((T*)a.out)[(long long)(row0 + t0 + t) * a.ldo + head * vdim + column] = from_float<T>(total);
        }
        // the next chunk's staging writes qs, fs and vs, which nobody reads any more; `partial` is written
        // again only behind the next barrier
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int d = g * R + j;
        if (live && d < dim) state[(long long)d * vdim + v] = S[j];
    }
}

template <typename T, int R>
int launch(const GatedRecurrenceArgs& a, cudaStream_t stream) {
    const size_t shared = (size_t)(2 * CHUNK * GROUPS * R + CHUNK * COLUMNS + CHUNK * GROUPS * COLUMNS) * sizeof(float);
    auto kernel = gated_recurrence_kernel<T, R>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    dim3 grid(a.seqs, a.heads, (a.vdim + COLUMNS - 1) / COLUMNS);
    return kidi_launch(kernel, grid, GROUPS * COLUMNS, shared, stream, a);
}

template <typename T>
int dispatch(const GatedRecurrenceArgs& a, cudaStream_t stream) {
    const int rows = (a.dim + GROUPS - 1) / GROUPS;
    if (rows <= 1) return launch<T, 1>(a, stream);
    if (rows <= 2) return launch<T, 2>(a, stream);
    if (rows <= 4) return launch<T, 4>(a, stream);
    if (rows <= 8) return launch<T, 8>(a, stream);
    if (rows <= 16) return launch<T, 16>(a, stream);
    if (rows <= 32) return launch<T, 32>(a, stream);
    return KIDI_REFUSED_SIZE;
}
}  // namespace

KIDI_API int kidi_gated_recurrence(const GatedRecurrenceArgs* args, int dtype, cudaStream_t stream) {
    const GatedRecurrenceArgs& a = *args;
    if (a.seqs <= 0) return 0;
    if (a.heads <= 0 || a.heads > 65535 || a.dim <= 0 || a.vdim <= 0 || (a.vdim + COLUMNS - 1) / COLUMNS > 65535)
        return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32) return dispatch<float>(a, stream);
    if (dtype == KIDI_BF16) return dispatch<bf16>(a, stream);
    return KIDI_REFUSED_DTYPE;
}

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
// tokens at a time are computed once a block into shared memory, a chunk ahead of the one being computed (its
// projections are loaded into registers before the current chunk's tokens are walked, so their latency hides
// behind the walk); the eight partial read-outs of a column meet in shared memory and are added in the order of g. A token's result therefore depends on the sizes only: not on
// what else is in the step, nor on how the sequence was cut into steps. The read-out leaves the kernel
// unnormalised (its columns lie in different blocks); the norm over vdim is a kernel of its own. For steps of many
// tokens q and f are computed once a row by a kernel of their own (into scratch memory), since every block of
// columns of a head would otherwise compute them again.
#include "common.cuh"
#include <type_traits>

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
    int rows;              // rows of the step (of qfv, out and gates)
    int narrow_blocks;     // the step brings many tokens a sequence: blocks of 16 columns when there are few blocks
    float* gates;          // [rows, 2*heads*dim] or null: scratch for q and f computed once a row by a kernel of
                           // their own (steps of many tokens), instead of once a block of columns inside the walk
};

namespace {
// A load that stays where it is written and hands back the bits as they are. The compiler would otherwise move a
// chunk's loads down to their first use, behind the walk over the chunk before it; and a conversion right behind a
// load makes the warp wait for it there, load after load. So a chunk's loads are issued together, their bits wait
// in registers, and they are converted where they are used.
template <typename T> struct Raw;
template <> struct Raw<float> {
    typedef float type;
    static __device__ __forceinline__ type load(const float* pointer) {
        float value;
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(value) : "l"(pointer));
        return value;
    }
    static __device__ __forceinline__ float value(type bits) { return bits; }
};
template <> struct Raw<bf16> {
    typedef unsigned short type;
    static __device__ __forceinline__ type load(const bf16* pointer) {
        unsigned short bits;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(bits) : "l"(pointer));
        return bits;
    }
    static __device__ __forceinline__ float value(type bits) { return __uint_as_float((unsigned)bits << 16); }
};

constexpr int THREADS = 256;
constexpr int CHUNK = 16;       // tokens whose gates are staged at a time

// COLUMNS: state columns of a block, one a lane of a group of COLUMNS lanes (32: a warp; 16: half a warp, for steps
// that would otherwise leave most SMs with one block or none); GROUPS = 256 / COLUMNS groups share the state's rows.
// q = silu(q~) and f = l + (1 - l) sigmoid(f~ + b) of every row, head and state row, once: [rows, 2*heads*dim].
template <typename T>
__global__ void recurrence_gates_kernel(GatedRecurrenceArgs a, long long total) {
    const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const int width = a.heads * a.dim;
    const long long row = index / width;
    const int c = (int)(index - row * width);
    const T* source = (const T*)a.qfv + row * a.ld;
    const float raw = to_float(source[c]);
    const float gate = 1.0f / (1.0f + expf(-(to_float(source[width + c]) + a.f_bias[c])));
    a.gates[row * 2 * width + c] = raw / (1.0f + expf(-raw));
    a.gates[row * 2 * width + width + c] = a.lower[c] + (1.0f - a.lower[c]) * gate;
}

// PRE: q and f come computed from `a.gates`.
template <typename T, int R, int COLUMNS, bool PRE>
__global__ void __launch_bounds__(THREADS) gated_recurrence_kernel(GatedRecurrenceArgs a) {
    extern __shared__ __align__(16) float shared[];
    typedef typename std::conditional<PRE, float, T>::type G;    // what the staged q and f are loaded as
    constexpr int GROUPS = THREADS / COLUMNS;
    constexpr int PADDED = GROUPS * R;                   // dim rounded up: rows beyond dim hold q = 0, f = 1
    constexpr int GATES = (CHUNK * PADDED + THREADS - 1) / THREADS;     // (q, f) pairs a thread stages a chunk
    constexpr int VALUES = CHUNK * COLUMNS / THREADS;
    const int seq = blockIdx.x, head = blockIdx.y;
    const int row0 = a.seq_row0[seq], count = a.seq_len[seq];
    if (count <= 0 || a.row_seq[row0] < 0) return;       // a padding sequence touches no state
    const int dim = a.dim, vdim = a.vdim;
    const int lane = threadIdx.x % COLUMNS, g = threadIdx.x / COLUMNS;
    const int v = blockIdx.z * COLUMNS + lane;
    const bool live = v < vdim;
    // two stages of (q, f, v) of CHUNK tokens, two of partial read-outs
    float* stage = shared;                               // [2][CHUNK][2 * PADDED + COLUMNS]
    constexpr int STAGE = CHUNK * (2 * PADDED + COLUMNS);
    float* partials = shared + 2 * STAGE;                // [2][CHUNK][GROUPS][COLUMNS]
    float* state = a.state + ((long long)a.seq_slot[seq] * a.heads + head) * dim * vdim;
    float S[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int d = g * R + j;
        S[j] = live && d < dim ? state[(long long)d * vdim + v] : 0.f;
    }
    // the bias and the lower bound of the gates this thread stages: the same rows d in every chunk
    float my_bias[GATES], my_lower[GATES];
#pragma unroll
    for (int i = 0; i < GATES; ++i) {
        const int d = (threadIdx.x + i * THREADS) % PADDED;
        my_bias[i] = d < dim ? a.f_bias[head * dim + d] : 0.f;
        my_lower[i] = d < dim ? a.lower[head * dim + d] : 0.f;
    }
    typename Raw<G>::type raw_q[GATES], raw_f[GATES];
    typename Raw<T>::type raw_v[VALUES];

    // the raw projections of the chunk that starts at token t0, into registers (all loads in flight together)
    auto fetch = [&](int t0) {
        const int tokens = min(CHUNK, count - t0);
#pragma unroll
        for (int i = 0; i < GATES; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / PADDED, d = index - t * PADDED;
            raw_q[i] = raw_f[i] = 0;
            if (t < tokens && d < dim) {
                if constexpr (PRE) {
                    const float* row = a.gates + (long long)(row0 + t0 + t) * 2 * a.heads * dim;
                    raw_q[i] = Raw<float>::load(row + head * dim + d);
                    raw_f[i] = Raw<float>::load(row + (a.heads + head) * dim + d);
                } else {
                    const T* row = (const T*)a.qfv + (long long)(row0 + t0 + t) * a.ld;
                    raw_q[i] = Raw<T>::load(row + head * dim + d);
                    raw_f[i] = Raw<T>::load(row + (a.heads + head) * dim + d);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < VALUES; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / COLUMNS, c = index - t * COLUMNS;
            const int column = blockIdx.z * COLUMNS + c;
            raw_v[i] = 0;
            if (t < tokens && column < vdim)
                raw_v[i] = Raw<T>::load((const T*)a.qfv + (long long)(row0 + t0 + t) * a.ld + 2 * a.heads * dim + head * vdim + column);
        }
    };
    // activations and gates of the fetched chunk, into a stage of shared memory
    auto put = [&](float* target) {
#pragma unroll
        for (int i = 0; i < GATES; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / PADDED, d = index - t * PADDED;
            if (index >= CHUNK * PADDED) continue;
            float q = 0.f, f = 1.f;
            if (d < dim) {
                if constexpr (PRE) {
                    q = raw_q[i];
                    f = raw_f[i];
                } else {
                    const float raw = Raw<T>::value(raw_q[i]);
                    q = raw / (1.0f + expf(-raw));
                    const float gate = 1.0f / (1.0f + expf(-(Raw<T>::value(raw_f[i]) + my_bias[i])));
                    f = my_lower[i] + (1.0f - my_lower[i]) * gate;
                }
            }
            target[t * (2 * PADDED + COLUMNS) + d] = q;
            target[t * (2 * PADDED + COLUMNS) + PADDED + d] = f;
        }
#pragma unroll
        for (int i = 0; i < VALUES; ++i) {
            const int index = threadIdx.x + i * THREADS, t = index / COLUMNS, c = index - t * COLUMNS;
            target[t * (2 * PADDED + COLUMNS) + 2 * PADDED + c] = Raw<T>::value(raw_v[i]);
        }
    };

    fetch(0);
    put(stage);
    __syncthreads();
    int turn = 0;
    for (int t0 = 0; t0 < count; t0 += CHUNK, turn ^= 1) {
        const int tokens = min(CHUNK, count - t0);
        const bool more = t0 + CHUNK < count;
        if (more) fetch(t0 + CHUNK);                     // on their way while this chunk is computed
        const float* current = stage + turn * STAGE;
        float* partial = partials + turn * (CHUNK * GROUPS * COLUMNS);
        for (int t = 0; t < tokens; ++t) {
            const float* q = current + t * (2 * PADDED + COLUMNS) + g * R;   // one address a warp: broadcasts
            const float* f = q + PADDED;
            const float value = current[t * (2 * PADDED + COLUMNS) + 2 * PADDED + lane];
            float sum = 0.f;
            if constexpr (R % 4 == 0) {
                float sums[4] = {0.f, 0.f, 0.f, 0.f};     // four chains instead of one of R links
#pragma unroll
                for (int j = 0; j < R; j += 4) {
                    const float4 f4 = *reinterpret_cast<const float4*>(f + j), q4 = *reinterpret_cast<const float4*>(q + j);
                    const float fj[4] = {f4.x, f4.y, f4.z, f4.w}, qj[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float s = fmaf(fj[e], S[j + e] - value, value);     // f S + (1 - f) v
                        S[j + e] = s;
                        sums[e] = fmaf(s, qj[e], sums[e]);
                    }
                }
                sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            } else {
#pragma unroll
                for (int j = 0; j < R; ++j) {
                    const float s = fmaf(f[j], S[j] - value, value);                  // f S + (1 - f) v
                    S[j] = s;
                    sum = fmaf(s, q[j], sum);
                }
            }
            partial[(t * GROUPS + g) * COLUMNS + lane] = sum;
        }
        if (more) put(stage + (turn ^ 1) * STAGE);
        __syncthreads();
        // (the stage and the partials written next are the other ones; these are free again behind the next barrier)
        for (int index = threadIdx.x; index < tokens * COLUMNS; index += THREADS) {
            const int t = index / COLUMNS, c = index - t * COLUMNS;
            const int column = blockIdx.z * COLUMNS + c;
            if (column >= vdim) continue;
            float total = 0.f;
#pragma unroll
            for (int k = 0; k < GROUPS; ++k) total += partial[(t * GROUPS + k) * COLUMNS + c];
            ((T*)a.out)[(long long)(row0 + t0 + t) * a.ldo + head * vdim + column] = from_float<T>(total);
        }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int d = g * R + j;
        if (live && d < dim) state[(long long)d * vdim + v] = S[j];
    }
}

template <typename T, int R, int COLUMNS, bool PRE>
int launch_form(const GatedRecurrenceArgs& a, cudaStream_t stream) {
    constexpr int GROUPS = THREADS / COLUMNS;
    const size_t shared = (size_t)2 * (CHUNK * (2 * GROUPS * R + COLUMNS) + CHUNK * GROUPS * COLUMNS) * sizeof(float);
    auto kernel = gated_recurrence_kernel<T, R, COLUMNS, PRE>;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    dim3 grid(a.seqs, a.heads, (a.vdim + COLUMNS - 1) / COLUMNS);
    return kidi_launch(kernel, grid, THREADS, shared, stream, a);
}

template <typename T, int R, int COLUMNS>
int launch(const GatedRecurrenceArgs& a, cudaStream_t stream) {
    if (!a.gates) return launch_form<T, R, COLUMNS, false>(a, stream);
    const long long total = (long long)a.rows * a.heads * a.dim;
    const int status = kidi_launch(recurrence_gates_kernel<T>, (unsigned)((total + 255) / 256), 256, 0, stream, a, total);
    return status ? status : launch_form<T, R, COLUMNS, true>(a, stream);
}

template <typename T, int COLUMNS>
int dispatch_rows(const GatedRecurrenceArgs& a, cudaStream_t stream) {
    const int rows = (a.dim + THREADS / COLUMNS - 1) / (THREADS / COLUMNS);
    if (rows <= 1) return launch<T, 1, COLUMNS>(a, stream);
    if (rows <= 2) return launch<T, 2, COLUMNS>(a, stream);
    if (rows <= 4) return launch<T, 4, COLUMNS>(a, stream);
    if (rows <= 8) return launch<T, 8, COLUMNS>(a, stream);
    if (rows <= 16) return launch<T, 16, COLUMNS>(a, stream);
    if (COLUMNS == 32 && rows <= 32) return launch<T, 32, 32>(a, stream);
    return KIDI_REFUSED_SIZE;
}

template <typename T>
int dispatch(const GatedRecurrenceArgs& a, cudaStream_t stream) {
    // Few (sequence, head, 32 columns) blocks: half as many columns a block, so that SMs hold two blocks or more.
    // The choice depends on the step's sizes only through the number of sequences; a row's result does not
    // depend on it beyond the order in which the partial read-outs are added.
    const long long blocks = (long long)a.seqs * a.heads * ((a.vdim + 31) / 32);
    if (a.narrow_blocks && blocks < 2 * 148 && a.vdim > 16) return dispatch_rows<T, 16>(a, stream);
    return dispatch_rows<T, 32>(a, stream);
}
}  // namespace

KIDI_API int kidi_gated_recurrence(const GatedRecurrenceArgs* args, int dtype, cudaStream_t stream) {
    const GatedRecurrenceArgs& a = *args;
    if (a.seqs <= 0) return 0;
    if (a.heads <= 0 || a.heads > 65535 || a.dim <= 0 || a.vdim <= 0 || (a.vdim + 15) / 16 > 65535)
        return KIDI_REFUSED_SIZE;
    if (dtype == KIDI_F32) return dispatch<float>(a, stream);
    if (dtype == KIDI_BF16) return dispatch<bf16>(a, stream);
    return KIDI_REFUSED_DTYPE;
}

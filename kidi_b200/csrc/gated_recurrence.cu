// A gated linear recurrence per head whose write strength is the complement of its forget gate (HGRN2):
//     q_t = silu(q~_t)                                  [dim]
//     f_t = l + (1 - l) * sigmoid(f~_t + b)             [dim]   l: a lower bound per channel
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T         [dim, vdim]
//     o_t = S_t^T q_t, divided by its root mean square over vdim and multiplied by a weight shared by the heads
// q~, f~, v are the columns of one fused projection [q~ | f~ | v]. The state S lives in 32-bit floats per cache
// slot and is carried from token to token; gates, state, read-out and the norm are 32-bit.
//
// One block per (sequence, head) walks the sequence's rows of the step in order. The state sits in shared memory;
// thread (v, g) owns column v of the rows d = g, g + G, ... and the G partial read-outs of a column are added in
// the order of g, so a token's result depends on the sizes only, not on what else is in the step.
#include "common.cuh"

struct GatedRecurrenceArgs {
    const void* qfv;       // [rows, ld]: heads*dim of q~, heads*dim of f~, heads*vdim of v
    long long ld;
    const float* f_bias;   // [heads*dim]
    const float* lower;    // [heads*dim]
    const float* norm;     // [vdim]
    float* state;          // [slots + 1, heads, dim, vdim]
    void* out;             // [rows, ldo]: heads*vdim
    long long ldo;
    const int* row_seq;    // [rows] (-1: padding)
    const int* seq_slot;   // [seqs]
    const int* seq_row0;   // [seqs]
    const int* seq_len;    // [seqs]
    int seqs, heads, dim, vdim, groups;
    float eps;
};

template <typename T>
__global__ void gated_recurrence_kernel(GatedRecurrenceArgs a) {
    extern __shared__ float shared[];
    const int seq = blockIdx.x, head = blockIdx.y;
    const int row0 = a.seq_row0[seq], count = a.seq_len[seq];
    if (count <= 0 || a.row_seq[row0] < 0) return;       // a padding sequence touches no state
    const int dim = a.dim, vdim = a.vdim, G = a.groups;
    const int columns = blockDim.x / G;                  // vdim rounded up to a multiple of 32
    const int v = threadIdx.x % columns, g = threadIdx.x / columns;
    float* S = shared;                                   // [dim][vdim]
    float* qs = S + dim * vdim;                          // [dim]
    float* fs = qs + dim;                                // [dim]
    float* partial = fs + dim;                           // [G][columns]
    float* readout = partial + G * columns;              // [columns]
    float* factor = readout + columns;                   // [1]
    float* state = a.state + ((long long)a.seq_slot[seq] * a.heads + head) * dim * vdim;
    for (int i = threadIdx.x; i < dim * vdim; i += blockDim.x) S[i] = state[i];
    const float* bias = a.f_bias + head * dim;
    const float* lower = a.lower + head * dim;
    for (int t = 0; t < count; ++t) {
        const T* row = (const T*)a.qfv + (long long)(row0 + t) * a.ld;
        __syncthreads();                                 // the state is loaded; the last token's read-out is stored
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            const float q = to_float(row[head * dim + d]);
            qs[d] = q / (1.0f + expf(-q));
            const float gate = 1.0f / (1.0f + expf(-(to_float(row[(a.heads + head) * dim + d]) + bias[d])));
            fs[d] = lower[d] + (1.0f - lower[d]) * gate;
        }
        __syncthreads();
        float sum = 0.f;
        if (v < vdim) {
            const float value = to_float(row[2 * a.heads * dim + head * vdim + v]);
            for (int d = g; d < dim; d += G) {
                const float f = fs[d];
                const float s = f * S[d * vdim + v] + (1.0f - f) * value;
                S[d * vdim + v] = s;
                sum = fmaf(s, qs[d], sum);
            }
        }
        partial[g * columns + v] = sum;
        __syncthreads();
        if (g == 0) {
            float total = 0.f;
            for (int k = 0; k < G; ++k) total += partial[k * columns + v];
            readout[v] = v < vdim ? total : 0.f;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            float square = 0.f;
            for (int c = threadIdx.x; c < columns; c += 32) square = fmaf(readout[c], readout[c], square);
            square = warp_sum(square);
            if (threadIdx.x == 0) factor[0] = 1.0f / sqrtf(square / (float)vdim + a.eps);
        }
        __syncthreads();
        if (g == 0 && v < vdim)
            ((T*)a.out)[(long long)(row0 + t) * a.ldo + head * vdim + v] = from_float<T>(readout[v] * factor[0] * a.norm[v]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < dim * vdim; i += blockDim.x) state[i] = S[i];
}

KIDI_API int kidi_gated_recurrence(const GatedRecurrenceArgs* args, int dtype, cudaStream_t stream) {
    GatedRecurrenceArgs a = *args;
    if (a.seqs <= 0) return 0;
    if (a.heads <= 0 || a.heads > 65535 || a.dim <= 0 || a.vdim <= 0 || a.vdim > 1024) return KIDI_REFUSED_SIZE;
    const int columns = (a.vdim + 31) / 32 * 32;
    int groups = 1;
    while (groups * 2 * columns <= 256 && groups * 2 <= a.dim) groups *= 2;
    a.groups = groups;
    const size_t shared = ((size_t)a.dim * a.vdim + 2 * a.dim + (groups + 1) * columns + 8) * sizeof(float);
    if (shared > 200 * 1024) return KIDI_REFUSED_SIZE;
    dim3 grid(a.seqs, a.heads);
    auto kernel = dtype == KIDI_F32 ? gated_recurrence_kernel<float> : gated_recurrence_kernel<bf16>;
    if (dtype != KIDI_F32 && dtype != KIDI_BF16) return KIDI_REFUSED_DTYPE;
    if (shared > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (status != cudaSuccess) return (int)status;
    }
    return kidi_launch(kernel, grid, groups * columns, shared, stream, a);
}

// y[M,N] = x[M,K] * W[N,K]^T with 32-bit multiply-add on the CUDA cores.
//
// This is the true 32-bit matrix product (no reduced-precision matrix mode) and the
// fallback for shapes the tensor-core kernels refuse. Every output element is one
// chain of fused multiply-adds over ascending k that starts from zero, so a row's
// result does not depend on how many other rows share the launch or on where the
// row falls in a tile. The reference's Linear is y = x W^T with W stored [out, in]
// (src/kidi/layers/linear.cpp:98-101,181-190).
#include "common.cuh"

namespace {
constexpr int TILE = 64;     // output tile is TILE x TILE
constexpr int TILE_K = 16;
constexpr int PAD = 4;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int M, int N, int K,
                 long long ldx, long long ldw, long long ldy, const float* __restrict__ bias, long long batch_x,
                 long long batch_w, long long batch_y) {
    // blockIdx.z: one product of a batch whose operands lie `batch_*` elements apart (0, 0, 0 without one)
    x += blockIdx.z * batch_x;
    w += blockIdx.z * batch_w;
    y += blockIdx.z * batch_y;
    __shared__ float xs[TILE_K][TILE + PAD];
    __shared__ float ws[TILE_K][TILE + PAD];
    const int tx = threadIdx.x & 15;   // 4 output columns (n) each
    const int ty = threadIdx.x >> 4;   // 4 output rows (m) each
    const int m0 = blockIdx.y * TILE, n0 = blockIdx.x * TILE;
    const int load_row = threadIdx.x >> 2;         // 0..63
    const int load_k = (threadIdx.x & 3) * 4;      // 0,4,8,12
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TILE_K) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + load_k + j;
            const int m = m0 + load_row, n = n0 + load_row;
            xs[load_k + j][load_row] = (m < M && k < K) ? to_float(x[m * ldx + k]) : 0.f;
            ws[load_k + j][load_row] = (n < N && k < K) ? to_float(w[n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TILE_K; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[m * ldy + n] = from_float<TY>(bias ? acc[i][j] + bias[n] : acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TY>
int launch(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy,
           const float* bias, cudaStream_t stream, int batch = 1, long long batch_x = 0, long long batch_w = 0,
           long long batch_y = 0) {
    dim3 grid((N + TILE - 1) / TILE, (M + TILE - 1) / TILE, batch);
    return kidi_launch(gemm_simt_kernel<TX, TW, TY>, grid, 256, 0, stream, (const TX*)x, (const TW*)w, (TY*)y, M, N, K,
                       ldx, ldw, ldy, bias, batch_x, batch_w, batch_y);
}
}  // namespace

// `bias` (float32 [N], or null) is added to every row after the chain of multiply-adds
// (the reference's Linear with bias, src/kidi/layers/linear.cpp:181-190).
KIDI_API int kidi_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int M, int N,
                            int K, long long ldx, long long ldw, long long ldy, const float* bias, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (M + TILE - 1) / TILE > 65535) return KIDI_REFUSED_SIZE;
#define KIDI_CASE(X, TX, W, TW, Y, TY)                                 \
    if (x_dtype == X && w_dtype == W && y_dtype == Y)                  \
        return launch<TX, TW, TY>(x, w, y, M, N, K, ldx, ldw, ldy, bias, stream);
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, KIDI_BF16, bf16)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

// The same for a batch of products (one per head, say): product b takes x + b * batch_x, w + b * batch_w and
// writes y + b * batch_y (strides in elements). Each output is the same ascending-k chain as above.
KIDI_API int kidi_gemm_simt_batched(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int M,
                                    int N, int K, long long ldx, long long ldw, long long ldy, int batch,
                                    long long batch_x, long long batch_w, long long batch_y, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || (M + TILE - 1) / TILE > 65535 || batch > 65535) return KIDI_REFUSED_SIZE;
#define KIDI_CASE(X, TX, W, TW, Y, TY)                                 \
    if (x_dtype == X && w_dtype == W && y_dtype == Y)                  \
        return launch<TX, TW, TY>(x, w, y, M, N, K, ldx, ldw, ldy, nullptr, stream, batch, batch_x, batch_w, batch_y);
    KIDI_CASE(KIDI_F32, float, KIDI_F32, float, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, KIDI_BF16, bf16)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_F32, float, KIDI_BF16, bf16, KIDI_F32, float)
    KIDI_CASE(KIDI_BF16, bf16, KIDI_F32, float, KIDI_BF16, bf16)
#undef KIDI_CASE
    return KIDI_REFUSED_DTYPE;
}

// The same batch of products for few rows (M <= 8): a warp computes y[0..M-1, n] of one product of the batch, its
// lanes striding k; the weight row is read once for all M rows. A row's result depends on K only.
namespace {
template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(128)
gemm_rows_batched_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int M, int N, int K,
                         long long ldx, long long ldw, long long ldy, long long batch_x, long long batch_w,
                         long long batch_y) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 4 + warp;
    if (n >= N) return;
    x += blockIdx.y * batch_x;
    w += blockIdx.y * batch_w + n * ldw;
    y += blockIdx.y * batch_y;
    float acc[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[m] = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float weight = to_float(w[k]);
#pragma unroll
        for (int m = 0; m < 8; ++m)
            if (m < M) acc[m] = fmaf(to_float(x[m * ldx + k]), weight, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const float total = warp_sum(acc[m]);
        if (lane == 0 && m < M) y[m * ldy + n] = from_float<TY>(total);
    }
}
}  // namespace

KIDI_API int kidi_gemm_rows_batched(const void* x, const void* w, void* y, int dtype, int M, int N, int K, long long ldx,
                                    long long ldw, long long ldy, int batch, long long batch_x, long long batch_w,
                                    long long batch_y, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || M > 8 || batch > 65535) return KIDI_REFUSED_SIZE;
    dim3 grid((N + 3) / 4, batch);
    if (dtype == KIDI_BF16)
        return kidi_launch(gemm_rows_batched_kernel<bf16, bf16, bf16>, grid, 128, 0, stream, (const bf16*)x, (const bf16*)w,
                           (bf16*)y, M, N, K, ldx, ldw, ldy, batch_x, batch_w, batch_y);
    if (dtype == KIDI_F32)
        return kidi_launch(gemm_rows_batched_kernel<float, float, float>, grid, 128, 0, stream, (const float*)x,
                           (const float*)w, (float*)y, M, N, K, ldx, ldw, ldy, batch_x, batch_w, batch_y);
    return KIDI_REFUSED_DTYPE;
}

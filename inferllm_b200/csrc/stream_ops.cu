// Small element-wise kernels between matrix products.
//
// gated_act:    out[t, i] = act(gu[t, 2i]) * gu[t, 2i + 1]  for the activations that the fused silu kernels do not
//               cover (act 1: silu, 2: relu, 3: tanh-form gelu); the packed projection holds gate and up of an
//               output next to each other, as in swiglu.cu.
// take_columns: y[t, :] = x[t, off : off + n] of a float32 matrix with row stride ld, as a contiguous matrix of
//               the activation dtype (what a second, low-rank product reads).
// join_rows:    y[t, :] = [a[t, :], b[t, :]] of two float32 matrices of equal width, in the activation dtype.
#include "common.cuh"

__device__ __forceinline__ float gate_act_of(float v, int act) {
    if (act == 1) return v / (1.0f + expf(-v));
    if (act == 2) return fmaxf(v, 0.f);
    if (act == 3) return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

template <typename TA>
__global__ void gated_act_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, long long n, int act) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / I;
    const int c = (int)(i - t * I);
    const float g = to_f32(gu[t * 2 * I + 2 * c]), u = to_f32(gu[t * 2 * I + 2 * c + 1]);
    out[i] = from_f32<TA>(gate_act_of(g, act) * u);
}

extern "C" int illm_gated_act(const void* gu, void* out, int act_dtype, int T, int I, int act, void* stream) {
    if (T <= 0 || I <= 0) return 0;
    if (act < 1 || act > 3) return ILLM_ERR_BAD_ARG;
    const long long n = (long long)T * I;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(gated_act_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, n, act);
    else if (act_dtype == ILLM_F32) illm_launch(gated_act_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, n, act);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

template <typename TA>
__global__ void take_columns_kernel(const float* __restrict__ x, int ld, int off, int n_cols, TA* __restrict__ y, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / n_cols;
    y[i] = from_f32<TA>(x[t * ld + off + (i - t * n_cols)]);
}

extern "C" int illm_take_columns(const float* x, int ld, int off, int n_cols, void* y, int act_dtype, int T, void* stream) {
    if (T <= 0 || n_cols <= 0) return 0;
    const long long n = (long long)T * n_cols;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(take_columns_kernel<bf16>, dim3(blocks), dim3(256), 0, s, x, ld, off, n_cols, (bf16*)y, n);
    else if (act_dtype == ILLM_F32) illm_launch(take_columns_kernel<float>, dim3(blocks), dim3(256), 0, s, x, ld, off, n_cols, (float*)y, n);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

template <typename TA>
__global__ void join_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, int H, TA* __restrict__ y, long long n) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / (2 * H);
    const int c = (int)(i - t * 2 * H);
    y[i] = from_f32<TA>(c < H ? a[t * H + c] : b[t * H + c - H]);
}

extern "C" int illm_join_rows(const float* a, const float* b, int H, void* y, int act_dtype, int T, void* stream) {
    if (T <= 0 || H <= 0) return 0;
    const long long n = (long long)T * 2 * H;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == ILLM_BF16) illm_launch(join_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, s, a, b, H, (bf16*)y, n);
    else if (act_dtype == ILLM_F32) illm_launch(join_rows_kernel<float>, dim3(blocks), dim3(256), 0, s, a, b, H, (float*)y, n);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

// Norm after the sum: the residual stream itself is replaced by the normed row.
//
//   v = alpha * x[r] + delta[r];   x[r] = v / sqrt(mean(v^2) + eps) * w;   y[r] = x[r] rounded to the compute dtype
//
// This is the arrangement "x <- norm(alpha * x + sublayer(x))": where add_rmsnorm (rmsnorm.cu) keeps the
// un-normed sum as the stream and hands the normed row to the next sublayer only, here the normed
// row is both.  The stream, the scaled sum, the mean of squares and the product with the weight are
// float32; w is float32 (a weight stored as an offset from one has the one added when it is loaded).
// The addend may also come as the unreduced K slices of a split matrix product (float32
// [splits, rows, H]); they are added in ascending order, as the stand-alone reduction would.
// One block per row and a fixed order of the sums, so a row's bits do not depend on the launch.
#include "common.cuh"

template <typename TD, typename TY>
__global__ void __launch_bounds__(1024)
scale_add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const float* __restrict__ w,
                         TY* __restrict__ y, int H, float alpha, float eps, const float* __restrict__ partials, int splits,
                         long long split_stride) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    float* x = resid + (size_t)blockIdx.x * H;
    const TD* dl = delta ? delta + (size_t)blockIdx.x * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = alpha * x[c];
        if (dl) v += to_f32(dl[c]);
        if (partials) {
            // the loads of eight slices are in flight together; the additions keep the slices' order
            const float* ps = partials + (size_t)blockIdx.x * H + c;
            float sum = 0.f;
            int k = 0;
            for (; k + 8 <= splits; k += 8) {
                float t[8];
#pragma unroll
                for (int u = 0; u < 8; u++) t[u] = ps[(size_t)(k + u) * split_stride];
#pragma unroll
                for (int u = 0; u < 8; u++) sum += t[u];
            }
            for (; k < splits; k++) sum += ps[(size_t)k * split_stride];
            v += sum;
        }
        x[c] = v;            // read again below by the same thread
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TY* o = y ? y + (size_t)blockIdx.x * H : nullptr;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = (x[c] * inv) * w[c];
        x[c] = v;
        if (o) o[c] = from_f32<TY>(v);
    }
}

extern "C" int illm_scale_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const float* w, void* y, int y_dtype,
                                      int n_rows, int H, float alpha, float eps, const float* partials, int splits, long long split_stride,
                                      void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || !resid || !w) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    // threads by the width alone, so a row's sums have the same order in every launch
    const int threads = H >= 4096 ? 1024 : H >= 1024 ? 512 : 256;
#define ILLM_PN(TD, TY) \
    illm_launch(scale_add_rmsnorm_kernel<TD, TY>, dim3(n_rows), dim3(threads), 0, s, resid, (const TD*)delta, w, (TY*)y, H, alpha, eps, partials, splits, \
                split_stride)
    if (delta_dtype == ILLM_F32 && y_dtype == ILLM_F32) ILLM_PN(float, float);
    else if (delta_dtype == ILLM_F32 && y_dtype == ILLM_BF16) ILLM_PN(float, bf16);
    else if (delta_dtype == ILLM_BF16 && y_dtype == ILLM_BF16) ILLM_PN(bf16, bf16);
    else if (delta_dtype == ILLM_BF16 && y_dtype == ILLM_F32) ILLM_PN(bf16, float);
    else return ILLM_ERR_BAD_ARG;
#undef ILLM_PN
    return illm_launch_status();
}

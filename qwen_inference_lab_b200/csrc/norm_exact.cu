// Root-mean-square norm whose arithmetic is float32 from end to end, for residual streams that are
// kept in float32 whatever the activation dtype is.
//
//   y = x / sqrt(mean(x^2) + eps) * (offset + w)
//
// Input and output types are independent (a float32 stream normed into bfloat16 rows for the
// products that follow); the statistics, the scaling and the weight multiply are float32 and the
// result is rounded once.  `offset` 1 serves weights that are stored around zero, 0 plain ones.
// With `rows` only those rows are normed, in that order.  The sum of squares is taken by a fixed
// tree over a fixed block size, so a row's result does not depend on the rest of the batch.
#include "common.cuh"

template <typename TI, typename TO, typename W>
__global__ void __launch_bounds__(256)
rmsnorm_exact_kernel(const TI* __restrict__ x, const W* __restrict__ weight, const int* __restrict__ rows,
                     TO* __restrict__ out, int width, float eps, float offset) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const int r = blockIdx.x;
    const TI* src = x + (size_t)(rows ? rows[r] : r) * width;
    TO* dst = out + (size_t)r * width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) {
        const float v = to_f32<TI>(src[i]);
        sq = fmaf(v, v, sq);
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += 256)
        dst[i] = from_f32<TO>(to_f32<TI>(src[i]) * scale * (offset + to_f32<W>(weight[i])));
}

extern "C" int qil_rmsnorm_exact(const void* x, int x_dtype, const void* weight, int weight_dtype, const int* rows,
                                 void* out, int out_dtype, int n_rows, int width, float eps, float offset,
                                 cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) QIL_REFUSE("rmsnorm_exact: width %d", width);
#define QIL_NORM_GO(TI, TO)                                                                                  \
    do {                                                                                                     \
        if (weight_dtype == QIL_F32)                                                                         \
            qil_launch_chained(rmsnorm_exact_kernel<TI, TO, float>, dim3(n_rows), dim3(256), 0, stream,      \
                               (const TI*)x, (const float*)weight, rows, (TO*)out, width, eps, offset);      \
        else                                                                                                 \
            qil_launch_chained(rmsnorm_exact_kernel<TI, TO, bf16>, dim3(n_rows), dim3(256), 0, stream,       \
                               (const TI*)x, (const bf16*)weight, rows, (TO*)out, width, eps, offset);       \
    } while (0)
    if (weight_dtype != QIL_F32 && weight_dtype != QIL_BF16) QIL_REFUSE("rmsnorm_exact: weight dtype %d", weight_dtype);
    if (x_dtype == QIL_F32 && out_dtype == QIL_F32) QIL_NORM_GO(float, float);
    else if (x_dtype == QIL_F32 && out_dtype == QIL_BF16) QIL_NORM_GO(float, bf16);
    else if (x_dtype == QIL_BF16 && out_dtype == QIL_BF16) QIL_NORM_GO(bf16, bf16);
    else if (x_dtype == QIL_BF16 && out_dtype == QIL_F32) QIL_NORM_GO(bf16, float);
    else QIL_REFUSE("rmsnorm_exact: dtypes %d -> %d", x_dtype, out_dtype);
#undef QIL_NORM_GO
    QIL_CHECK_LAUNCH();
}

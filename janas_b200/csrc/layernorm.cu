// Layer norm with weight and bias over the rows of the float32 residual stream,
// with the residual add of what the layer before left fused in front of it.
//
//   x  <-  x + m * (sum_s a[s] + sum_s b[s])          (in place, when a is given)
//   out =  (x - mean) / sqrt(var + eps) * w + bias     var = mean((x - mean)^2)
//
// a and b are two stacks of partial sums (a mixer's and a feed-forward's result
// over the same input, for a layer whose sublayers run side by side); m is the
// factor on the residual branch.  One block per row; the row stays in shared
// memory between the add, the two sums and the output, so x and the partial sums
// are read once.  Mean and variance are two passes over the row in float32 (the
// variance of the deviations, not E[x^2] - mean^2), and the order of the
// additions depends only on the row's width: a row's bits are the same in any
// batch.
#include "common.cuh"
#include "kernels.h"

namespace jb {

template <typename TO>
__global__ void __launch_bounds__(256)
layernorm_kernel(float *__restrict__ x, const float *__restrict__ a, int Sa, size_t a_stride,
                 const float *__restrict__ b, int Sb, size_t b_stride, float mult,
                 const int32_t *__restrict__ row_idx, const float *__restrict__ w,
                 const float *__restrict__ bias, TO *__restrict__ out, int dm, float eps)
{
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_trigger();
    int r = blockIdx.x;
    pdl_wait();
    size_t src = row_idx != nullptr ? (size_t)row_idx[r] : (size_t)r;
    float *xr = x + src * dm;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < dm; i += blockDim.x) {
        float v = xr[i];
        if (a != nullptr) {
            float d = add_partials(0.0f, a + src * dm + i, Sa, a_stride);
            if (b != nullptr)
                d += add_partials(0.0f, b + src * dm + i, Sb, b_stride);
            v = fmaf(mult, d, v);
            xr[i] = v;
        }
        row[i] = v;
        sum += v;
    }
    if (out == nullptr)
        return;
    float mean = block_sum(sum, red) / (float)dm;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < dm; i += blockDim.x) {
        float d = row[i] - mean;
        sq = fmaf(d, d, sq);
    }
    float var = block_sum(sq, red) / (float)dm;
    float inv = 1.0f / sqrtf(var + eps);
    TO *o = out + (size_t)r * dm;
    for (int i = threadIdx.x; i < dm; i += blockDim.x)
        o[i] = from_f<TO>(fmaf((row[i] - mean) * inv, w[i], bias != nullptr ? bias[i] : 0.0f));
}

}  // namespace jb

using namespace jb;

// x: float32 [n, dm], updated in place when a is given (b only together with a).
// row_idx (n_out int32, or null): the rows to normalize; with row_idx no add is
// done.  w, bias: float32 [dm] (bias may be null).  out null: the add alone.
extern "C" int jb_layernorm(float *x, const float *a, int Sa, long long a_stride, const float *b,
                            int Sb, long long b_stride, float mult, const int32_t *row_idx,
                            const float *w, const float *bias, void *out, int out_dt, int n_out,
                            int dm, float eps, cudaStream_t st)
{
    if (n_out <= 0)
        return JB_OK;
    if (dm <= 0 || dm > 49152 / 4 || (a == nullptr && b != nullptr) || (a != nullptr && row_idx != nullptr) ||
        (out != nullptr && w == nullptr) || (a != nullptr && Sa <= 0) || (b != nullptr && Sb <= 0))
        return JB_EINVAL;
    unsigned threads = (unsigned)min(256, (dm + 31) / 32 * 32);
    size_t smem = (size_t)dm * 4;
    if (out == nullptr || out_dt == JB_F32)
        launch(layernorm_kernel<float>, n_out, threads, smem, st, x, a, Sa, (size_t)a_stride, b, Sb,
               (size_t)b_stride, mult, row_idx, w, bias, (float *)out, dm, eps);
    else if (out_dt == JB_BF16)
        launch(layernorm_kernel<bf16>, n_out, threads, smem, st, x, a, Sa, (size_t)a_stride, b, Sb,
               (size_t)b_stride, mult, row_idx, w, bias, (bf16 *)out, dm, eps);
    else
        return JB_EINVAL;
    return launch_status();
}

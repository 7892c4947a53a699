// Element-wise kernels of layers whose norms need no sum over the row: the
// Dynamic Tanh norm, the sigmoid gate on a sublayer's result, both of them fused
// with the residual add, the PolyNorm activation (which does sum over the row),
// the embedding gather with a learned position vector, and a plain scaling.
//
//   dyt(v)      = tanh(alpha v) w + b                 alpha a scalar, w and b vectors
//   gated(y, g) = (sum_s y_s + by) / (1 + exp(-(sum_s g_s + bg)))
//   polynorm(z) = c0 n(z) + c1 n(z^2) + c2 n(z^3) + c3,  n(u) = u / sqrt(mean(u^2) + eps)
//
// Everything is computed in float; the small parameter vectors (w, b, alpha, the
// biases, the four coefficients) are float arrays.  A product's result arrives
// as a stack of S partial sums that are added in the order 0 .. S-1.  A row's
// result depends on nothing but the row (PolyNorm's sums run in an order that
// depends on the row's width alone), so it is the same bits in any batch.
#include "common.cuh"
#include "kernels.h"

namespace jb {

template <typename TT, typename TP>
__global__ void embed_pos_kernel(const TT *__restrict__ table, const TP *__restrict__ pos_table,
                                 const int32_t *__restrict__ tokens,
                                 const int32_t *__restrict__ row_pos, float *__restrict__ x, int dm)
{
    pdl_trigger();
    pdl_wait();
    size_t row = blockIdx.x;
    const TT *src = table + (size_t)tokens[row] * dm;
    const TP *ps = pos_table + (size_t)row_pos[row] * dm;
    float *dst = x + row * dm;
    for (int i = threadIdx.x; i < dm; i += blockDim.x)
        dst[i] = to_f(src[i]) + to_f(ps[i]);
}

__device__ __forceinline__ float dyt1(float v, float alpha, float w, float b)
{
    return fmaf(tanhf(alpha * v), w, b);
}

__device__ __forceinline__ float sigmoid1(float v) { return 1.0f / (1.0f + expf(-v)); }

// x: [n, dm] float, updated in place when delta is given (x += sum of delta's S
// partial sums).  row_idx (or null) picks the rows that are normed; out has one
// row per picked row.  One thread per value.
template <typename TO>
__global__ void dyt_kernel(float *__restrict__ x, const float *__restrict__ delta, int S,
                           size_t delta_stride, const int32_t *__restrict__ row_idx,
                           const float *__restrict__ w, const float *__restrict__ b,
                           const float *__restrict__ alpha, TO *__restrict__ out, int dm,
                           size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t orow = i / dm;
    int c = (int)(i - orow * dm);
    float wv = w[c], bv = b[c], a = alpha[0];
    pdl_wait();
    size_t row = row_idx ? (size_t)row_idx[orow] : orow;
    float v = x[row * dm + c];
    if (delta) {
        v = add_partials(v, delta + row * dm + c, S, delta_stride);
        x[row * dm + c] = v;
    }
    out[i] = from_f<TO>(dyt1(v, a, wv, bv));
}

// out[n, dm] float = (sum_s y_s + y_bias) * sigmoid(sum_s g_s + g_bias).  The gate's
// values are columns g_col0 .. g_col0 + dm - 1 of rows g_ld wide (the gate may be
// part of a wider product).
__global__ void gate_mul_kernel(const float *__restrict__ y, int Sy, size_t y_stride,
                                const float *__restrict__ y_bias, const float *__restrict__ g,
                                int Sg, size_t g_stride, int g_ld, int g_col0,
                                const float *__restrict__ g_bias, float *__restrict__ out, int dm,
                                size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t row = i / dm;
    int c = (int)(i - row * dm);
    float yb = y_bias ? y_bias[c] : 0.0f, gb = g_bias ? g_bias[c] : 0.0f;
    pdl_wait();
    float yv = add_partials(0.0f, y + i, Sy, y_stride) + yb;
    float gv = add_partials(0.0f, g + row * g_ld + g_col0 + c, Sg, g_stride) + gb;
    out[i] = yv * sigmoid1(gv);
}

// A whole sublayer's end in one pass over the row:
//   x += dyt_post(gated(y, g));   out = dyt_next(x)   (when a next norm is given)
template <typename TO>
__global__ void gated_dyt_residual_kernel(
    float *__restrict__ x, const float *__restrict__ y, int Sy, size_t y_stride,
    const float *__restrict__ y_bias, const float *__restrict__ g, int Sg, size_t g_stride,
    int g_ld, int g_col0, const float *__restrict__ g_bias, const float *__restrict__ pw,
    const float *__restrict__ pb, const float *__restrict__ palpha, const float *__restrict__ nw,
    const float *__restrict__ nb, const float *__restrict__ nalpha, TO *__restrict__ out, int dm,
    size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t row = i / dm;
    int c = (int)(i - row * dm);
    float yb = y_bias ? y_bias[c] : 0.0f, gb = g_bias ? g_bias[c] : 0.0f;
    float pwv = pw[c], pbv = pb[c], pa = palpha[0];
    float nwv = 0.0f, nbv = 0.0f, na = 0.0f;
    if (out != nullptr) {
        nwv = nw[c];
        nbv = nb[c];
        na = nalpha[0];
    }
    pdl_wait();
    float yv = add_partials(0.0f, y + i, Sy, y_stride) + yb;
    float gv = add_partials(0.0f, g + row * g_ld + g_col0 + c, Sg, g_stride) + gb;
    float v = x[i] + dyt1(yv * sigmoid1(gv), pa, pwv, pbv);
    x[i] = v;
    if (out != nullptr)
        out[i] = from_f<TO>(dyt1(v, na, nwv, nbv));
}

// z: S stacked partial sums, rows z_ld wide of which the first ff columns are the
// feed-forward's values.  One block per row; the three sums of powers are added in
// an order that depends on ff alone.
template <typename TO>
__global__ void polynorm_kernel(const float *__restrict__ z, int S, size_t stride, int z_ld,
                                const float *__restrict__ coef, float eps, TO *__restrict__ out,
                                int ff)
{
    __shared__ float red[32];
    pdl_trigger();
    float c0 = coef[0], c1 = coef[1], c2 = coef[2], c3 = coef[3];
    pdl_wait();
    size_t row = blockIdx.x;
    const float *zr = z + row * z_ld;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int i = threadIdx.x; i < ff; i += blockDim.x) {
        float v = add_partials(0.0f, zr + i, S, stride);
        float v2 = v * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v2 * v, v2 * v, s6);
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    float r1 = 1.0f / sqrtf(s2 / (float)ff + eps);
    float r2 = 1.0f / sqrtf(s4 / (float)ff + eps);
    float r3 = 1.0f / sqrtf(s6 / (float)ff + eps);
    TO *o = out + row * ff;
    for (int i = threadIdx.x; i < ff; i += blockDim.x) {
        float v = add_partials(0.0f, zr + i, S, stride);
        float v2 = v * v;
        o[i] = from_f<TO>(c0 * (v * r1) + c1 * (v2 * r2) + c2 * (v2 * v * r3) + c3);
    }
}

__global__ void scale_kernel(float *__restrict__ x, float s, size_t total)
{
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total)
        x[i] *= s;
}

__global__ void add_bias_kernel(float *__restrict__ y, const float *__restrict__ bias, int m,
                                size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    float b = bias[i % m];
    pdl_wait();
    y[i] += b;
}

// The fused [q | k | v] product's sums plus its bias: q rows out, K and V into the
// cache pages at each row's position.  Widths: nh hd, nkv hd, nkv vd; without
// `append` the product holds q alone.
template <typename TC>
__global__ void qkv_bias_append_kernel(const float *__restrict__ qkv, int S, size_t stride, int ld,
                                       const float *__restrict__ bias,
                                       const int32_t *__restrict__ row_pos,
                                       const int32_t *__restrict__ row_seq,
                                       const int32_t *__restrict__ block_table, int bt_stride,
                                       TC *__restrict__ q_out, TC *__restrict__ k_cache,
                                       TC *__restrict__ v_cache, int nh, int nkv, int hd, int vd,
                                       int width, size_t total)
{
    pdl_trigger();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t row = i / width;
    int c = (int)(i - row * width);
    float bv = bias ? bias[c] : 0.0f;
    pdl_wait();
    float v = add_partials(0.0f, qkv + row * ld + c, S, stride) + bv;
    int qw = nh * hd, kw = nkv * hd;
    if (c < qw) {
        q_out[row * qw + c] = from_f<TC>(v);
        return;
    }
    int pos = row_pos[row];
    int page = block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE];
    if (c < qw + kw) {
        int kc = c - qw, h = kc / hd, d = kc - h * hd;
        k_cache[(((size_t)page * nkv + h) * PAGE + pos % PAGE) * hd + d] = from_f<TC>(v);
    } else {
        int vc = c - qw - kw, h = vc / vd, d = vc - h * vd;
        v_cache[(((size_t)page * nkv + h) * PAGE + pos % PAGE) * vd + d] = from_f<TC>(v);
    }
}

static int row_threads(int width)
{
    int t = 32;
    while (t < 1024 && t * 8 < width)
        t <<= 1;
    return t;
}

}  // namespace jb

using namespace jb;

extern "C" int jb_embed_pos(const void *table, int table_dt, const void *pos_table, int pos_dt,
                            const int32_t *tokens, const int32_t *row_pos, float *x, int n, int dm,
                            cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    int threads = row_threads(dm);
#define JB_EP(TT, TP)                                                                         \
    launch(embed_pos_kernel<TT, TP>, n, threads, 0, st, (const TT *)table, (const TP *)pos_table, \
           tokens, row_pos, x, dm)
    if (table_dt == JB_F32 && pos_dt == JB_F32)
        JB_EP(float, float);
    else if (table_dt == JB_BF16 && pos_dt == JB_BF16)
        JB_EP(bf16, bf16);
    else if (table_dt == JB_F32 && pos_dt == JB_BF16)
        JB_EP(float, bf16);
    else if (table_dt == JB_BF16 && pos_dt == JB_F32)
        JB_EP(bf16, float);
    else
        return JB_EINVAL;
#undef JB_EP
    return launch_status();
}

extern "C" int jb_dyt(float *x, const float *delta, int S, long long delta_stride,
                      const int32_t *row_idx, const float *w, const float *b, const float *alpha,
                      void *out, int out_dt, int n_out, int dm, cudaStream_t st)
{
    size_t total = (size_t)n_out * dm;
    if (total == 0)
        return JB_OK;
    if (delta && row_idx)
        return JB_EINVAL;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dt == JB_F32)
        launch(dyt_kernel<float>, blocks, 256, 0, st, x, delta, S, (size_t)delta_stride, row_idx, w,
               b, alpha, (float *)out, dm, total);
    else if (out_dt == JB_BF16)
        launch(dyt_kernel<bf16>, blocks, 256, 0, st, x, delta, S, (size_t)delta_stride, row_idx, w,
               b, alpha, (bf16 *)out, dm, total);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_gate_mul(const float *y, int Sy, long long y_stride, const float *y_bias,
                           const float *g, int Sg, long long g_stride, int g_ld, int g_col0,
                           const float *g_bias, float *out, int n, int dm, cudaStream_t st)
{
    size_t total = (size_t)n * dm;
    if (total == 0)
        return JB_OK;
    launch(gate_mul_kernel, (unsigned)((total + 255) / 256), 256, 0, st, y, Sy, (size_t)y_stride,
           y_bias, g, Sg, (size_t)g_stride, g_ld, g_col0, g_bias, out, dm, total);
    return launch_status();
}

extern "C" int jb_gated_dyt_residual(float *x, const float *y, int Sy, long long y_stride,
                                     const float *y_bias, const float *g, int Sg,
                                     long long g_stride, int g_ld, int g_col0, const float *g_bias,
                                     const float *pw, const float *pb, const float *palpha,
                                     const float *nw, const float *nb, const float *nalpha,
                                     void *out, int out_dt, int n, int dm, cudaStream_t st)
{
    size_t total = (size_t)n * dm;
    if (total == 0)
        return JB_OK;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (out == nullptr || out_dt == JB_F32)
        launch(gated_dyt_residual_kernel<float>, blocks, 256, 0, st, x, y, Sy, (size_t)y_stride,
               y_bias, g, Sg, (size_t)g_stride, g_ld, g_col0, g_bias, pw, pb, palpha, nw, nb, nalpha,
               (float *)out, dm, total);
    else if (out_dt == JB_BF16)
        launch(gated_dyt_residual_kernel<bf16>, blocks, 256, 0, st, x, y, Sy, (size_t)y_stride,
               y_bias, g, Sg, (size_t)g_stride, g_ld, g_col0, g_bias, pw, pb, palpha, nw, nb, nalpha,
               (bf16 *)out, dm, total);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_polynorm(const float *z, int S, long long stride, int z_ld, const float *coef,
                           float eps, void *out, int out_dt, int n, int ff, cudaStream_t st)
{
    if (n <= 0 || ff <= 0)
        return JB_OK;
    int threads = row_threads(ff);
    if (out_dt == JB_F32)
        launch(polynorm_kernel<float>, n, threads, 0, st, z, S, (size_t)stride, z_ld, coef, eps,
               (float *)out, ff);
    else if (out_dt == JB_BF16)
        launch(polynorm_kernel<bf16>, n, threads, 0, st, z, S, (size_t)stride, z_ld, coef, eps,
               (bf16 *)out, ff);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_scale(float *x, float s, long long total, cudaStream_t st)
{
    if (total <= 0)
        return JB_OK;
    launch(scale_kernel, (unsigned)((total + 255) / 256), 256, 0, st, x, s, (size_t)total);
    return launch_status();
}

extern "C" int jb_add_bias(float *y, const float *bias, int n, int m, cudaStream_t st)
{
    size_t total = (size_t)n * m;
    if (total == 0)
        return JB_OK;
    launch(add_bias_kernel, (unsigned)((total + 255) / 256), 256, 0, st, y, bias, m, total);
    return launch_status();
}

extern "C" int jb_qkv_bias_append(const float *qkv, int S, long long stride, int ld,
                                  const float *bias, const int32_t *row_pos,
                                  const int32_t *row_seq, const int32_t *block_table,
                                  int bt_stride, void *q_out, void *k_cache, void *v_cache,
                                  int cache_dt, int n, int nh, int nkv, int hd, int vd, int append,
                                  cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    if (nh <= 0 || hd <= 0 || (append && (nkv <= 0 || vd <= 0 || !k_cache || !v_cache)))
        return JB_EINVAL;
    int width = nh * hd + (append ? nkv * (hd + vd) : 0);
    if (ld < width)
        return JB_EINVAL;
    size_t total = (size_t)n * width;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (cache_dt == JB_F32)
        launch(qkv_bias_append_kernel<float>, blocks, 256, 0, st, qkv, S, (size_t)stride, ld, bias,
               row_pos, row_seq, block_table, bt_stride, (float *)q_out, (float *)k_cache,
               (float *)v_cache, nh, nkv, hd, vd, width, total);
    else if (cache_dt == JB_BF16)
        launch(qkv_bias_append_kernel<bf16>, blocks, 256, 0, st, qkv, S, (size_t)stride, ld, bias,
               row_pos, row_seq, block_table, bt_stride, (bf16 *)q_out, (bf16 *)k_cache,
               (bf16 *)v_cache, nh, nkv, hd, vd, width, total);
    else
        return JB_EINVAL;
    return launch_status();
}

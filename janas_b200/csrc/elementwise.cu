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

// The same two with the hardware's exponential and reciprocal, for the bfloat16
// path: absolute error of a few 1e-7 (tanh(t) = 1 - 2 / (1 + e^(2t))), far below
// what that path's stored activations round to.  FAST false: the library functions.
template <bool FAST> __device__ __forceinline__ float tanh_f(float t)
{
    if (!FAST)
        return tanhf(t);
    float e = __expf(2.0f * fminf(t, 40.0f));
    return 1.0f - __fdividef(2.0f, 1.0f + e);
}
template <bool FAST> __device__ __forceinline__ float dyt_f(float v, float alpha, float w, float b)
{
    return fmaf(tanh_f<FAST>(alpha * v), w, b);
}
template <bool FAST> __device__ __forceinline__ float sigmoid_f(float v)
{
    if (!FAST)
        return 1.0f / (1.0f + expf(-v));
    return __fdividef(1.0f, 1.0f + __expf(-fmaxf(v, -80.0f)));
}

// Four neighbouring columns' sums of S partial sums, added in the order 0 .. S-1
// (the same order as add_partials), eight partial sums fetched together.
__device__ __forceinline__ float4 sum_partials4(const float *__restrict__ p, int S, size_t stride)
{
    // one partial sum (every product of many rows): nothing to add, and no loop whose
    // bookkeeping would cost more than the kernels around it do
    if (S == 1)
        return load4(p);
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s0 = 0; s0 < S; s0 += 8) {
        float4 t[8];
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (s0 + u < S)
                t[u] = load4(p + (size_t)(s0 + u) * stride);
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (s0 + u < S) {
                v.x += t[u].x; v.y += t[u].y; v.z += t[u].z; v.w += t[u].w;
            }
    }
    return v;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b)
{
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

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

// The same with four neighbouring columns per thread (dm, the gate's row length and
// first column multiples of 4, everything at 16-byte boundaries).
// Grid: x over groups of GDR_ROWS rows, y over blocks of columns (no division per
// thread); with two rows a thread fetches its columns' parameters once for both and
// has both rows' values in flight together (many rows); with one, more threads share
// the work (few rows, many partial sums).
template <typename TO, bool FAST, int GDR_ROWS>
__global__ void __launch_bounds__(256)
gated_dyt_residual_vec_kernel(
    float *__restrict__ x, const float *__restrict__ y, int Sy, size_t y_stride,
    const float *__restrict__ y_bias, const float *__restrict__ g, int Sg, size_t g_stride,
    int g_ld, int g_col0, const float *__restrict__ g_bias, const float *__restrict__ pw,
    const float *__restrict__ pb, const float *__restrict__ palpha, const float *__restrict__ nw,
    const float *__restrict__ nb, const float *__restrict__ nalpha, TO *__restrict__ out, int dm,
    int n)
{
    pdl_trigger();
    size_t row0 = (size_t)blockIdx.x * GDR_ROWS;
    int c = (int)(blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= dm)
        return;
    float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 yb = y_bias ? load4(y_bias + c) : zero, gb = g_bias ? load4(g_bias + c) : zero;
    float4 pwv = load4(pw + c), pbv = load4(pb + c);
    float pa = palpha[0];
    float4 nwv = zero, nbv = zero;
    float na = 0.0f;
    if (out != nullptr) {
        nwv = load4(nw + c);
        nbv = load4(nb + c);
        na = nalpha[0];
    }
    pdl_wait();
    float4 xs[GDR_ROWS], ys[GDR_ROWS], gs[GDR_ROWS];
#pragma unroll
    for (int r = 0; r < GDR_ROWS; r++) {
        size_t row = row0 + r;
        if (row < (size_t)n) {
            size_t i = row * dm + c;
            xs[r] = load4(x + i);
            ys[r] = sum_partials4(y + i, Sy, y_stride);
            gs[r] = sum_partials4(g + row * g_ld + g_col0 + c, Sg, g_stride);
        }
    }
#pragma unroll
    for (int r = 0; r < GDR_ROWS; r++) {
        size_t row = row0 + r;
        if (row >= (size_t)n)
            break;
        size_t i = row * dm + c;
        float4 xv = xs[r], yv = add4(ys[r], yb), gv = add4(gs[r], gb);
        xv.x += dyt_f<FAST>(yv.x * sigmoid_f<FAST>(gv.x), pa, pwv.x, pbv.x);
        xv.y += dyt_f<FAST>(yv.y * sigmoid_f<FAST>(gv.y), pa, pwv.y, pbv.y);
        xv.z += dyt_f<FAST>(yv.z * sigmoid_f<FAST>(gv.z), pa, pwv.z, pbv.z);
        xv.w += dyt_f<FAST>(yv.w * sigmoid_f<FAST>(gv.w), pa, pwv.w, pbv.w);
        store4(x + i, xv);
        if (out != nullptr)
            store4(out + i,
                   make_float4(dyt_f<FAST>(xv.x, na, nwv.x, nbv.x), dyt_f<FAST>(xv.y, na, nwv.y, nbv.y),
                               dyt_f<FAST>(xv.z, na, nwv.z, nbv.z), dyt_f<FAST>(xv.w, na, nwv.w, nbv.w)));
    }
}

__device__ __forceinline__ void power_sums(float4 v, float &s2, float &s4, float &s6)
{
    float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        float v2 = e[k] * e[k], v3 = v2 * e[k];
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
}

__device__ __forceinline__ float4 poly4(float4 v, float c0, float c1, float c2, float c3, float r1,
                                        float r2, float r3)
{
    float e[4] = {v.x, v.y, v.z, v.w}, o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        float v2 = e[k] * e[k];
        o[k] = c0 * (e[k] * r1) + c1 * (v2 * r2) + c2 * (v2 * e[k] * r3) + c3;
    }
    return make_float4(o[0], o[1], o[2], o[3]);
}

// Three sums over a block at once; every thread gets them.  red: 96 floats.
__device__ __forceinline__ void block_sum3(float &a, float &b, float &c, float *red)
{
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int nwarp = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    c = warp_sum(c);
    __syncthreads();
    if (lane == 0) {
        red[warp] = a;
        red[32 + warp] = b;
        red[64 + warp] = c;
    }
    __syncthreads();
    a = warp_sum(lane < nwarp ? red[lane] : 0.0f);
    b = warp_sum(lane < nwarp ? red[32 + lane] : 0.0f);
    c = warp_sum(lane < nwarp ? red[64 + lane] : 0.0f);
}

// PolyNorm with the row held in registers: a block of up to 512 threads per row,
// KEEP groups of four neighbouring values per thread (ff a multiple of 4, up to
// 16,384), one pass over memory, two blocks to an SM.  The sums run in an order
// that depends on ff alone.
template <typename TO, int KEEP>
__global__ void __launch_bounds__(512, 2)
polynorm_vec_kernel(const float *__restrict__ z, int S, size_t stride, int z_ld,
                    const float *__restrict__ coef, float eps, TO *__restrict__ out, int ff)
{
    __shared__ float red[96];
    pdl_trigger();
    float c0 = coef[0], c1 = coef[1], c2 = coef[2], c3 = coef[3];
    pdl_wait();
    size_t row = blockIdx.x;
    const float *zr = z + row * z_ld;
    int nv = ff / 4;
    float4 v[KEEP];
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
#pragma unroll
    for (int u = 0; u < KEEP; u++) {
        int j = threadIdx.x + u * blockDim.x;
        v[u] = j < nv ? sum_partials4(zr + 4 * j, S, stride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        power_sums(v[u], s2, s4, s6);
    }
    block_sum3(s2, s4, s6, red);
    float r1 = 1.0f / sqrtf(s2 / (float)ff + eps);
    float r2 = 1.0f / sqrtf(s4 / (float)ff + eps);
    float r3 = 1.0f / sqrtf(s6 / (float)ff + eps);
    TO *o = out + row * ff;
#pragma unroll
    for (int u = 0; u < KEEP; u++) {
        int j = threadIdx.x + u * blockDim.x;
        if (j < nv)
            store4(o + 4 * j, poly4(v[u], c0, c1, c2, c3, r1, r2, r3));
    }
}

// PolyNorm for few rows, bfloat16 out: a row is shared out among the C CTAs of a
// cluster (per4 groups of four values each, one group per thread), so that all a
// row needs is fetched at once; the CTAs' three sums meet through distributed
// shared memory and are added in rank order by everyone.
template <int C>
__global__ void __launch_bounds__(1024)
polynorm_cluster_kernel(const float *__restrict__ z, int S, size_t stride, int z_ld,
                        const float *__restrict__ coef, float eps, bf16 *__restrict__ out, int ff,
                        int per4)
{
    __shared__ float red[96];
    __shared__ float shares[3][C];     // shares[k][r]: written here by the CTA of rank r
    pdl_trigger();
    float c0 = coef[0], c1 = coef[1], c2 = coef[2], c3 = coef[3];
    uint32_t rank = cluster_rank();
    size_t row = blockIdx.x / C;
    int nv = ff / 4;
    int j = (int)rank * per4 + threadIdx.x;
    bool mine = (int)threadIdx.x < per4 && j < nv;
    pdl_wait();
    const float *zr = z + row * z_ld;
    float4 v = mine ? sum_partials4(zr + 4 * j, S, stride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    power_sums(v, s2, s4, s6);
    block_sum3(s2, s4, s6, red);
    if (threadIdx.x < C) {
        cluster_write(&shares[0][rank], threadIdx.x, s2);
        cluster_write(&shares[1][rank], threadIdx.x, s4);
        cluster_write(&shares[2][rank], threadIdx.x, s6);
    }
    cluster_arrive();
    cluster_wait();
    float t2 = 0.0f, t4 = 0.0f, t6 = 0.0f;
#pragma unroll
    for (int r = 0; r < C; r++) {
        t2 += shares[0][r];
        t4 += shares[1][r];
        t6 += shares[2][r];
    }
    float r1 = 1.0f / sqrtf(t2 / (float)ff + eps);
    float r2 = 1.0f / sqrtf(t4 / (float)ff + eps);
    float r3 = 1.0f / sqrtf(t6 / (float)ff + eps);
    if (mine)
        store4(out + row * ff + 4 * j, poly4(v, c0, c1, c2, c3, r1, r2, r3));
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

// A factor on the queries that grows with the position p in steps of `every`
// positions: 1 + coef * ln(floor((p + 1) / every) + 1).
__device__ __forceinline__ float query_temperature(int pos, float coef, int every)
{
    return 1.0f + coef * logf((float)((pos + 1) / every) + 1.0f);
}

// The fused [q | k | v] product's sums plus its bias: q rows out, K and V into the
// cache pages at each row's position.  With q_every > 0 the queries are multiplied
// by query_temperature() of their row's position.  Widths: nh hd, nkv hd, nkv vd; without
// `append` the product holds q alone.
template <typename TC>
__global__ void qkv_bias_append_kernel(const float *__restrict__ qkv, int S, size_t stride, int ld,
                                       const float *__restrict__ bias,
                                       const int32_t *__restrict__ row_pos,
                                       const int32_t *__restrict__ row_seq,
                                       const int32_t *__restrict__ block_table, int bt_stride,
                                       TC *__restrict__ q_out, TC *__restrict__ k_cache,
                                       TC *__restrict__ v_cache, int nh, int nkv, int hd, int vd,
                                       int width, size_t total, float q_coef, int q_every)
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
        if (q_every > 0)
            v *= query_temperature(row_pos[row], q_coef, q_every);
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

// The same with four neighbouring columns per thread (hd and vd multiples of 4: the
// four never straddle two heads), for ROWS rows each (grid: x over groups of rows, y
// over blocks of columns).
template <typename TC, int ROWS>
__global__ void __launch_bounds__(256)
qkv_bias_append_vec_kernel(const float *__restrict__ qkv, int S, size_t stride, int ld,
                           const float *__restrict__ bias, const int32_t *__restrict__ row_pos,
                           const int32_t *__restrict__ row_seq,
                           const int32_t *__restrict__ block_table, int bt_stride,
                           TC *__restrict__ q_out, TC *__restrict__ k_cache,
                           TC *__restrict__ v_cache, int nh, int nkv, int hd, int vd, int width,
                           int n, float q_coef, int q_every)
{
    pdl_trigger();
    size_t row0 = (size_t)blockIdx.x * ROWS;
    int c = (int)(blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= width)
        return;
    float4 bv = bias ? load4(bias + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int qw = nh * hd, kw = nkv * hd;
    // where this thread's four values go within a row of q, or within a head of the cache
    bool is_q = c < qw, is_k = !is_q && c < qw + kw;
    int h = 0, d = 0;
    if (is_k) {
        h = (c - qw) / hd;
        d = (c - qw) - h * hd;
    } else if (!is_q) {
        h = (c - qw - kw) / vd;
        d = (c - qw - kw) - h * vd;
    }
    int pos[ROWS], page[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
        pos[r] = page[r] = 0;
        if (!is_q && row0 + r < (size_t)n) {
            pos[r] = row_pos[row0 + r];
            page[r] = block_table[(size_t)row_seq[row0 + r] * bt_stride + pos[r] / PAGE];
        } else if (q_every > 0 && row0 + r < (size_t)n) {
            pos[r] = row_pos[row0 + r];
        }
    }
    pdl_wait();
    float4 v[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; r++)
        if (row0 + r < (size_t)n)
            v[r] = sum_partials4(qkv + (row0 + r) * ld + c, S, stride);
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
        size_t row = row0 + r;
        if (row >= (size_t)n)
            break;
        float4 o = add4(v[r], bv);
        if (is_q && q_every > 0) {
            float t = query_temperature(pos[r], q_coef, q_every);
            o = make_float4(o.x * t, o.y * t, o.z * t, o.w * t);
        }
        if (is_q)
            store4(q_out + row * qw + c, o);
        else if (is_k)
            store4(k_cache + (((size_t)page[r] * nkv + h) * PAGE + pos[r] % PAGE) * hd + d, o);
        else
            store4(v_cache + (((size_t)page[r] * nkv + h) * PAGE + pos[r] % PAGE) * vd + d, o);
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
                                     void *out, int out_dt, int n, int dm, int fast,
                                     cudaStream_t st)
{
    size_t total = (size_t)n * dm;
    if (total == 0)
        return JB_OK;
    auto al16 = [](const void *p) { return (uintptr_t)p % 16 == 0; };
    if (dm % 4 == 0 && g_ld % 4 == 0 && g_col0 % 4 == 0 && y_stride % 4 == 0 && g_stride % 4 == 0 &&
        al16(x) && al16(y) && al16(g) && al16(y_bias) && al16(g_bias) && al16(pw) && al16(pb) &&
        al16(nw) && al16(nb) && (uintptr_t)out % 8 == 0 && (out == nullptr || out_dt == JB_F32 ||
                                                             out_dt == JB_BF16)) {
        // blocks that the row's groups of four fill without idle threads, where that can be
        unsigned threads = (unsigned)min(256, (dm / 4 + 31) / 32 * 32);
        if (dm / 4 > 256 && (dm / 4) % 128 == 0 && (dm / 4) % 256 != 0)
            threads = 128;
        // the bfloat16 path (fast says so: the last layer's call has no norm output
        // to tell it by) takes the hardware's exponential
        int rows_per = n >= 64 ? 2 : 1;
        dim3 grid((unsigned)((n + rows_per - 1) / rows_per), (unsigned)((dm / 4 + threads - 1) / threads));
#define JB_GDR(TO, F, R)                                                                      \
    launch(gated_dyt_residual_vec_kernel<TO, F, R>, grid, threads, 0, st, x, y, Sy,            \
           (size_t)y_stride, y_bias, g, Sg, (size_t)g_stride, g_ld, g_col0, g_bias, pw, pb,    \
           palpha, nw, nb, nalpha, (TO *)out, dm, n)
#define JB_GDR_R(TO, F)                                                                       \
    do {                                                                                       \
        if (rows_per == 2)                                                                     \
            JB_GDR(TO, F, 2);                                                                  \
        else                                                                                   \
            JB_GDR(TO, F, 1);                                                                  \
    } while (0)
        if (fast && (out == nullptr || out_dt == JB_BF16)) {
            JB_GDR_R(bf16, true);
        } else if (out == nullptr || out_dt == JB_F32) {
            if (!al16(out))
                return JB_EINVAL;
            JB_GDR_R(float, false);
        } else {
            JB_GDR_R(bf16, false);
        }
#undef JB_GDR
#undef JB_GDR_R
        return launch_status();
    }
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
    bool vec = ff % 4 == 0 && z_ld % 4 == 0 && stride % 4 == 0 && (uintptr_t)z % 16 == 0 &&
               (uintptr_t)out % (out_dt == JB_F32 ? 16 : 8) == 0;
    // few rows of the bfloat16 path: a cluster of eight CTAs per row
    if (vec && out_dt == JB_BF16 && n <= 32 && ff >= 2048 && ff <= 8 * 4 * 1024) {
        constexpr int C = 8;
        int per4 = (ff / 4 + C - 1) / C;
        unsigned threads = (unsigned)((per4 + 31) / 32 * 32);
        launch_cluster(polynorm_cluster_kernel<C>, dim3((unsigned)n * C), threads, 0, st, C, z, S,
                       (size_t)stride, z_ld, coef, eps, (bf16 *)out, ff, per4);
        return launch_status();
    }
    if (vec && ff <= 8 * 4 * 512 && (out_dt == JB_F32 || out_dt == JB_BF16)) {
        int nv = ff / 4;
        // threads and values per thread depend on ff alone
        int keep = nv <= 512 ? 1 : (nv + 511) / 512;
        unsigned threads = (unsigned)(((nv + keep - 1) / keep + 31) / 32 * 32);
#define JB_PN(TO, K)                                                                          \
    launch(polynorm_vec_kernel<TO, K>, n, threads, 0, st, z, S, (size_t)stride, z_ld, coef, eps, \
           (TO *)out, ff)
#define JB_PNK(TO)                                                                            \
    do {                                                                                       \
        if (keep == 1)                                                                         \
            JB_PN(TO, 1);                                                                      \
        else if (keep == 2)                                                                    \
            JB_PN(TO, 2);                                                                      \
        else if (keep == 3)                                                                    \
            JB_PN(TO, 3);                                                                      \
        else if (keep == 4)                                                                    \
            JB_PN(TO, 4);                                                                      \
        else if (keep == 5)                                                                    \
            JB_PN(TO, 5);                                                                      \
        else if (keep == 6)                                                                    \
            JB_PN(TO, 6);                                                                      \
        else if (keep == 7)                                                                    \
            JB_PN(TO, 7);                                                                      \
        else                                                                                   \
            JB_PN(TO, 8);                                                                      \
    } while (0)
        if (out_dt == JB_F32)
            JB_PNK(float);
        else
            JB_PNK(bf16);
#undef JB_PN
#undef JB_PNK
        return launch_status();
    }
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
    return jb_qkv_bias_append_temp(qkv, S, stride, ld, bias, row_pos, row_seq, block_table, bt_stride,
                                   q_out, k_cache, v_cache, cache_dt, n, nh, nkv, hd, vd, append,
                                   0.0f, 0, st);
}

// The same with a query temperature: with q_every > 0 every query value of a row at
// position p is multiplied by 1 + q_coef * ln(floor((p + 1) / q_every) + 1).
extern "C" int jb_qkv_bias_append_temp(const float *qkv, int S, long long stride, int ld,
                                       const float *bias, const int32_t *row_pos,
                                       const int32_t *row_seq, const int32_t *block_table,
                                       int bt_stride, void *q_out, void *k_cache, void *v_cache,
                                       int cache_dt, int n, int nh, int nkv, int hd, int vd,
                                       int append, float q_coef, int q_every, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    // nh = 0 with append: the product holds keys and values alone
    if (nh < 0 || (nh == 0 && !append) || hd <= 0 || (append && (nkv <= 0 || vd <= 0 || !k_cache || !v_cache)))
        return JB_EINVAL;
    int width = nh * hd + (append ? nkv * (hd + vd) : 0);
    if (ld < width)
        return JB_EINVAL;
    size_t total = (size_t)n * width;
    size_t esz = cache_dt == JB_F32 ? 4 : 2;
    if (hd % 4 == 0 && (!append || vd % 4 == 0) && ld % 4 == 0 && stride % 4 == 0 &&
        (uintptr_t)qkv % 16 == 0 && (uintptr_t)bias % 16 == 0 && (uintptr_t)q_out % (4 * esz) == 0 &&
        (uintptr_t)k_cache % (4 * esz) == 0 && (uintptr_t)v_cache % (4 * esz) == 0 &&
        (cache_dt == JB_F32 || cache_dt == JB_BF16)) {
        unsigned threads = (unsigned)min(256, (width / 4 + 31) / 32 * 32);
        int rows_per = n >= 64 ? 2 : 1;
        dim3 grid((unsigned)((n + rows_per - 1) / rows_per), (unsigned)((width / 4 + threads - 1) / threads));
#define JB_APP(TC, R)                                                                         \
    launch(qkv_bias_append_vec_kernel<TC, R>, grid, threads, 0, st, qkv, S, (size_t)stride, ld, \
           bias, row_pos, row_seq, block_table, bt_stride, (TC *)q_out, (TC *)k_cache,         \
           (TC *)v_cache, nh, nkv, hd, vd, width, n, q_coef, q_every)
        if (cache_dt == JB_F32 && rows_per == 2)
            JB_APP(float, 2);
        else if (cache_dt == JB_F32)
            JB_APP(float, 1);
        else if (rows_per == 2)
            JB_APP(bf16, 2);
        else
            JB_APP(bf16, 1);
#undef JB_APP
        return launch_status();
    }
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (cache_dt == JB_F32)
        launch(qkv_bias_append_kernel<float>, blocks, 256, 0, st, qkv, S, (size_t)stride, ld, bias,
               row_pos, row_seq, block_table, bt_stride, (float *)q_out, (float *)k_cache,
               (float *)v_cache, nh, nkv, hd, vd, width, total, q_coef, q_every);
    else if (cache_dt == JB_BF16)
        launch(qkv_bias_append_kernel<bf16>, blocks, 256, 0, st, qkv, S, (size_t)stride, ld, bias,
               row_pos, row_seq, block_table, bt_stride, (bf16 *)q_out, (bf16 *)k_cache,
               (bf16 *)v_cache, nh, nkv, hd, vd, width, total, q_coef, q_every);
    else
        return JB_EINVAL;
    return launch_status();
}

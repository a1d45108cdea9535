// Layer norm (mean and variance over a row, weight and bias) around the residual add, for
// blocks that norm a sublayer's RESULT and feed the next sublayer the stream itself:
//
//   x   = resid[row] (+ LN_post(delta[row]))        -- the pending norm of the update, then the add
//   resid[row] = x                                   -- unless rows are selected
//   out = LN_pre(x)  or  x                           -- the next reader's input, in its dtype
//
// Every step is optional.  All arithmetic is float32; the variance is the mean of the squared
// deviations from the mean (two passes over the row, which is held in shared memory).  One block
// a row; the order of the additions depends only on the block size, so a row does not depend on
// the batch.
#include "common.cuh"

#define LN_THREADS 256

template <typename T>
__global__ void __launch_bounds__(LN_THREADS) ln_add_norm_kernel(
    float* __restrict__ resid, int ldr, const T* __restrict__ delta, int ldd,
    const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps,
    const float* __restrict__ pre_w, const float* __restrict__ pre_b, float pre_eps,
    T* __restrict__ out, int ldo, const int* __restrict__ rows, int dim) {
    extern __shared__ float ln_smem[];
    __shared__ float scratch[33];
    float* xs = ln_smem;
    float* ds = ln_smem + dim;
    pdl_wait();
    pdl_launch_dependents();
    const int row = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    const int tid = threadIdx.x;
    float* rr = resid + (size_t)row * ldr;
    for (int i = tid; i < dim; i += LN_THREADS) xs[i] = rr[i];
    if (delta != nullptr) {
        const T* dr = delta + (size_t)row * ldd;
        float s = 0.f;
        for (int i = tid; i < dim; i += LN_THREADS) {
            const float v = to_float(dr[i]);
            ds[i] = v;
            s += v;
        }
        const float mean = block_sum(s, scratch) / (float)dim;
        float q = 0.f;
        for (int i = tid; i < dim; i += LN_THREADS) {
            const float c = ds[i] - mean;
            q += c * c;
        }
        const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)dim + post_eps);
        for (int i = tid; i < dim; i += LN_THREADS) {
            float v = (ds[i] - mean) * rstd;
            if (post_w != nullptr) v = v * post_w[i] + post_b[i];
            xs[i] += v;
        }
        if (rows == nullptr)
            for (int i = tid; i < dim; i += LN_THREADS) rr[i] = xs[i];
    }
    if (out == nullptr) return;
    T* orow = out + (size_t)blockIdx.x * ldo;
    if (pre_w == nullptr) {
        for (int i = tid; i < dim; i += LN_THREADS) orow[i] = from_float<T>(xs[i]);
        return;
    }
    float s = 0.f;
    for (int i = tid; i < dim; i += LN_THREADS) s += xs[i];
    const float mean = block_sum(s, scratch) / (float)dim;
    float q = 0.f;
    for (int i = tid; i < dim; i += LN_THREADS) {
        const float c = xs[i] - mean;
        q += c * c;
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)dim + pre_eps);
    for (int i = tid; i < dim; i += LN_THREADS)
        orow[i] = from_float<T>((xs[i] - mean) * rstd * pre_w[i] + pre_b[i]);
}

template <typename T>
static int launch_ln(float* resid, int ldr, const T* delta, int ldd, const float* post_w,
                     const float* post_b, float post_eps, const float* pre_w, const float* pre_b,
                     float pre_eps, T* out, int ldo, const int* rows, int n_rows, int dim,
                     cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (dim <= 0 || resid == nullptr || (post_w == nullptr) != (post_b == nullptr) ||
        (pre_w == nullptr) != (pre_b == nullptr))
        return SLB_ERR_BAD_ARG;
    const size_t smem = (size_t)2 * dim * sizeof(float);
    if (smem > 200 * 1024) return SLB_ERR_TOO_LARGE;
    static unsigned long long configured = 0;
    const int e = slb_configure(&configured, ln_add_norm_kernel<T>, 200 * 1024);
    if (e != 0) return e;
    return slb_launch(ln_add_norm_kernel<T>, dim3(n_rows), dim3(LN_THREADS), smem, st, resid, ldr,
                      delta, ldd, post_w, post_b, post_eps, pre_w, pre_b, pre_eps, out, ldo, rows, dim);
}

extern "C" {
int slb_ln_add_norm_f32(float* resid, int ldr, const float* delta, int ldd, const float* post_w,
                        const float* post_b, float post_eps, const float* pre_w, const float* pre_b,
                        float pre_eps, float* out, int ldo, const int* rows, int n_rows, int dim,
                        cudaStream_t st) {
    return launch_ln<float>(resid, ldr, delta, ldd, post_w, post_b, post_eps, pre_w, pre_b, pre_eps,
                            out, ldo, rows, n_rows, dim, st);
}
int slb_ln_add_norm_bf16(float* resid, int ldr, const bf16* delta, int ldd, const float* post_w,
                         const float* post_b, float post_eps, const float* pre_w, const float* pre_b,
                         float pre_eps, bf16* out, int ldo, const int* rows, int n_rows, int dim,
                         cudaStream_t st) {
    return launch_ln<bf16>(resid, ldr, delta, ldd, post_w, post_b, post_eps, pre_w, pre_b, pre_eps,
                           out, ldo, rows, n_rows, dim, st);
}
}

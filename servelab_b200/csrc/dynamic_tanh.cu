// Dynamic Tanh norm fused with the residual add around it.
//
// y = tanh(alpha * x) * w + b per element (alpha a learned scalar): no mean, no variance,
// no root mean square, so a row needs no reduction and the kernel is a plain elementwise
// pass over the float32 residual stream.  One launch does up to three things for a row:
//
//   d      = post != null ? tanh(post_alpha * delta) * post_w + post_b : delta
//            (the norm on a sublayer's RESULT, applied before the result is added)
//   resid += d                     (in place, float32; skipped when rows are selected)
//   out    = tanh(alpha * resid) * w + b   (the norm on the NEXT sublayer's input)
//
// All arithmetic is float32; `delta` and `out` have the compute type T.  The scalars are
// read from device memory, so the launch takes no value from the host.
#include "common.cuh"

template <typename T, int VEC>
__global__ void __launch_bounds__(256) dyt_add_norm_kernel(
    float* __restrict__ resid, int ldr, const T* __restrict__ delta, int ldd,
    const float* __restrict__ post_alpha, const float* __restrict__ post_w,
    const float* __restrict__ post_b, const float* __restrict__ alpha,
    const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ out, int ldo,
    const int* __restrict__ row_map, int dim) {
    const float pa = post_alpha != nullptr ? *post_alpha : 0.f;      // (weights: before the wait)
    const float a = alpha != nullptr ? *alpha : 0.f;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y;
    const int src = row_map != nullptr ? row_map[r] : r;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c0 >= dim) return;
    float x[VEC];
    float* rp = resid + (size_t)src * ldr + c0;
    if constexpr (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(rp);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
        x[0] = rp[0];
    }
    if (delta != nullptr) {
        const T* dp = delta + (size_t)src * ldd + c0;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            float d = to_float(dp[i]);
            if (post_alpha != nullptr) d = tanhf(pa * d) * post_w[c0 + i] + post_b[c0 + i];
            x[i] += d;
        }
        if (row_map == nullptr) {
            if constexpr (VEC == 4) *reinterpret_cast<float4*>(rp) = make_float4(x[0], x[1], x[2], x[3]);
            else rp[0] = x[0];
        }
    }
    if (out != nullptr) {
        T* op = out + (size_t)r * ldo + c0;
#pragma unroll
        for (int i = 0; i < VEC; ++i) op[i] = from_float<T>(tanhf(a * x[i]) * w[c0 + i] + b[c0 + i]);
    }
}

template <typename T>
static int launch_dyt(float* resid, int ldr, const T* delta, int ldd, const float* post_alpha,
                      const float* post_w, const float* post_b, const float* alpha, const float* w,
                      const float* b, T* out, int ldo, const int* row_map, int rows, int dim,
                      cudaStream_t st) {
    if (rows <= 0) return 0;
    if (dim <= 0 || resid == nullptr || rows > 65535 * 1024) return SLB_ERR_BAD_ARG;
    if (out != nullptr && (alpha == nullptr || w == nullptr || b == nullptr)) return SLB_ERR_BAD_ARG;
    if (post_alpha != nullptr && (post_w == nullptr || post_b == nullptr || delta == nullptr)) return SLB_ERR_BAD_ARG;
    if (rows > 65535) return SLB_ERR_TOO_LARGE;
    const bool vec = dim % 4 == 0 && ldr % 4 == 0 && ((uintptr_t)resid & 15) == 0;
    if (vec) {
        const dim3 grid((dim / 4 + 255) / 256, rows);
        return slb_launch(dyt_add_norm_kernel<T, 4>, grid, dim3(256), 0, st, resid, ldr, delta, ldd,
                          post_alpha, post_w, post_b, alpha, w, b, out, ldo, row_map, dim);
    }
    const dim3 grid((dim + 255) / 256, rows);
    return slb_launch(dyt_add_norm_kernel<T, 1>, grid, dim3(256), 0, st, resid, ldr, delta, ldd,
                      post_alpha, post_w, post_b, alpha, w, b, out, ldo, row_map, dim);
}

extern "C" {
int slb_dyt_add_norm_f32(float* resid, int ldr, const float* delta, int ldd, const float* post_alpha,
                         const float* post_w, const float* post_b, const float* alpha, const float* w,
                         const float* b, float* out, int ldo, const int* row_map, int rows, int dim,
                         cudaStream_t st) {
    return launch_dyt<float>(resid, ldr, delta, ldd, post_alpha, post_w, post_b, alpha, w, b, out, ldo,
                             row_map, rows, dim, st);
}
int slb_dyt_add_norm_bf16(float* resid, int ldr, const bf16* delta, int ldd, const float* post_alpha,
                          const float* post_w, const float* post_b, const float* alpha, const float* w,
                          const float* b, bf16* out, int ldo, const int* row_map, int rows, int dim,
                          cudaStream_t st) {
    return launch_dyt<bf16>(resid, ldr, delta, ldd, post_alpha, post_w, post_b, alpha, w, b, out, ldo,
                            row_map, rows, dim, st);
}
}

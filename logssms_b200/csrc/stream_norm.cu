// Norms of a residual stream that is kept in 32-bit whatever the activation dtype (post-norm layers).
//
//   skip_rmsnorm : v = skip * x + y (+ row_scale[t] * extra);  n = v / sqrt(mean(v^2) + eps) * w
//                  out_f32 = n (the new stream), out_act = n rounded to the activation dtype (what the next
//                  sublayer's products read).  x is float32, y and extra are activations.  Without y it is the
//                  plain RMSNorm of the stream (the norm in front of the output head).
#include "lb200/common.cuh"
using namespace lb200;

template <typename T>
__global__ void skip_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ y, const T* __restrict__ extra,
                                    const float* __restrict__ row_scale, float skip, const float* __restrict__ weight,
                                    float eps, float* out_f32, T* __restrict__ out_act, int H) {
    extern __shared__ float row[];          // H floats
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    const float rs = (extra != nullptr) ? row_scale[blockIdx.x] : 0.f;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = skip * x[base + c];
        if (y != nullptr) v += to_f32(y[base + c]);
        if (extra != nullptr) v += rs * to_f32(extra[base + c]);
        row[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float n = row[c] * inv * weight[c];
        if (out_f32 != nullptr) out_f32[base + c] = n;
        if (out_act != nullptr) out_act[base + c] = from_f32<T>(n);
    }
}

extern "C" int lb_skip_rmsnorm(const float* x, const void* y, const void* extra, const float* row_scale, float skip,
                               const float* weight, float eps, float* out_f32, void* out_act, int rows, int H, int dtype,
                               void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || (size_t)H * sizeof(float) > 160 * 1024) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(skip_rmsnorm_kernel<T>, smem, have);
        skip_rmsnorm_kernel<T><<<rows, threads, smem, (cudaStream_t)stream>>>(
            x, (const T*)y, (const T*)extra, row_scale, skip, weight, eps, out_f32, (T*)out_act, H);
    });
    return launch_status();
}

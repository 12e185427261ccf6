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

// the same for bfloat16 activations and a width that is a multiple of 4: 16-byte pieces of the stream, 8-byte pieces of
// the activations, the row kept in registers between the two passes (up to 4 pieces per thread)
constexpr int kVecPieces = 4;
__global__ void __launch_bounds__(256) skip_rmsnorm_vec_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                                               const __nv_bfloat16* __restrict__ extra, const float* __restrict__ row_scale,
                                                               float skip, const float* __restrict__ weight, float eps, float* out_f32,
                                                               __nv_bfloat16* __restrict__ out_act, int H) {
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    const float rs = (extra != nullptr) ? row_scale[blockIdx.x] : 0.f;
    float4 v[kVecPieces];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kVecPieces; ++u) {
        const int c = (threadIdx.x + u * 256) * 4;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < H) {
            const float4 xv = *reinterpret_cast<const float4*>(x + base + c);
            v[u] = make_float4(skip * xv.x, skip * xv.y, skip * xv.z, skip * xv.w);
            if (y != nullptr) {
                const uint2 yv = *reinterpret_cast<const uint2*>(y + base + c);
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.y));
                v[u].x += a.x; v[u].y += a.y; v[u].z += b.x; v[u].w += b.y;
            }
            if (extra != nullptr) {
                const uint2 ev = *reinterpret_cast<const uint2*>(extra + base + c);
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ev.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ev.y));
                v[u].x += rs * a.x; v[u].y += rs * a.y; v[u].z += rs * b.x; v[u].w += rs * b.y;
            }
            ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int u = 0; u < kVecPieces; ++u) {
        const int c = (threadIdx.x + u * 256) * 4;
        if (c < H) {
            const float4 w = *reinterpret_cast<const float4*>(weight + c);
            const float4 n = make_float4(v[u].x * inv * w.x, v[u].y * inv * w.y, v[u].z * inv * w.z, v[u].w * inv * w.w);
            if (out_f32 != nullptr) *reinterpret_cast<float4*>(out_f32 + base + c) = n;
            if (out_act != nullptr) {
                uint2 o;
                *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(n.x, n.y);
                *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(n.z, n.w);
                *reinterpret_cast<uint2*>(out_act + base + c) = o;
            }
        }
    }
}

extern "C" int lb_skip_rmsnorm(const float* x, const void* y, const void* extra, const float* row_scale, float skip,
                               const float* weight, float eps, float* out_f32, void* out_act, int rows, int H, int dtype,
                               void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || (size_t)H * sizeof(float) > 160 * 1024) return kBadSize;
    const uintptr_t all = (uintptr_t)x | (uintptr_t)y | (uintptr_t)extra | (uintptr_t)weight | (uintptr_t)out_f32 | (uintptr_t)out_act;
    if (dtype == kBF16 && H % 4 == 0 && H <= 256 * 4 * kVecPieces && (all & 15) == 0) {
        skip_rmsnorm_vec_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)extra, row_scale,
                                                                       skip, weight, eps, out_f32, (__nv_bfloat16*)out_act, H);
        return launch_status();
    }
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

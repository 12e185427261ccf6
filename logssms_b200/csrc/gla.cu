// Gated linear attention with a decay per key channel, token by token.
//
//   a_t[d]  = sigmoid(z_t[d]) ^ (1 / tau)            (32-bit: log-sigmoid, division by tau, exponential)
//   S_t     = diag(a_t) S_{t-1} + k_t v_t^T            (S: [key channels, value channels] per head, 32-bit)
//   o_t     = S_t^T (q_t * q_scale)
//
//  gla_scan      : the recurrence over every request's tokens of a step, state read from and written back to the
//                  request's slot (a request that starts at position 0 starts from zeros whatever the slot holds).
//                  A CTA owns (request, head, a tile of value channels); a thread owns R state rows of one value
//                  column, DS threads of a warp share a column.  q, k, the decays and v of 8 tokens at a time are
//                  staged in shared memory, so the inner loop touches registers and shared memory only.
//  gla_norm_gate : y = o / sqrt(mean_head(o^2) + eps) * w[c] * silu(g), o in 32-bit, w shared by the heads.
#include "lb200/common.cuh"
using namespace lb200;

constexpr int kGlaTokens = 8;

__device__ __forceinline__ float log_sigmoid(float z) {
    return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}

template <typename T, int R, int DS>
__global__ void gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long row_stride,
                                const float* __restrict__ z, float* __restrict__ o, float* state,
                                const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
                                const int* __restrict__ request_list, int H, int dim, int vdim, float inv_tau, float q_scale) {
    constexpr int DP = R * DS;                       // key channels, padded
    extern __shared__ float sm[];
    const int cols = blockDim.x / DS;
    float* qs = sm;                                  // [kGlaTokens][DP]
    float* ks = qs + kGlaTokens * DP;
    float* as = ks + kGlaTokens * DP;
    float* vs = as + kGlaTokens * DP;                // [kGlaTokens][cols]
    const int b = request_list ? request_list[blockIdx.z] : blockIdx.z;
    if (b < 0) return;
    const int h = blockIdx.y;
    const int col_local = threadIdx.x / DS, s = threadIdx.x % DS;
    const int c = blockIdx.x * cols + col_local;
    const int first = cu[b], last = cu[b + 1];
    const size_t sbase = ((size_t)slots[b] * H + h) * dim * vdim;
    const bool fresh = start_pos[b] == 0;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = s * R + r;
        S[r] = (!fresh && d < dim && c < vdim) ? state[sbase + (size_t)d * vdim + c] : 0.f;
    }
    for (int t0 = first; t0 < last; t0 += kGlaTokens) {
        const int n = min(kGlaTokens, last - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < n * DP; i += blockDim.x) {
            const int tt = i / DP, d = i % DP;
            float qv = 0.f, kv = 0.f, av = 0.f;
            if (d < dim) {
                const size_t row = (size_t)(t0 + tt);
                qv = to_f32(q[row * row_stride + h * dim + d]) * q_scale;
                kv = to_f32(k[row * row_stride + h * dim + d]);
                av = expf(log_sigmoid(z[(row * H + h) * dim + d]) * inv_tau);
            }
            qs[i] = qv; ks[i] = kv; as[i] = av;
        }
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, cc = blockIdx.x * cols + i % cols;
            vs[i] = cc < vdim ? to_f32(v[(size_t)(t0 + tt) * row_stride + h * vdim + cc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vv = vs[tt * cols + col_local];
            const float* qr = qs + tt * DP + s * R;
            const float* kr = ks + tt * DP + s * R;
            const float* ar = as + tt * DP + s * R;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                S[r] = ar[r] * S[r] + kr[r] * vv;
                acc += qr[r] * S[r];
            }
#pragma unroll
            for (int off = 1; off < DS; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (s == 0 && c < vdim) o[((size_t)(t0 + tt) * H + h) * vdim + c] = acc;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = s * R + r;
        if (d < dim && c < vdim) state[sbase + (size_t)d * vdim + c] = S[r];
    }
}

template <typename T, int R, int DS>
static int launch_gla_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, float* o, float* state,
                           const int* cu, const int* start_pos, const int* slots, const int* request_list, int num_requests,
                           int H, int dim, int vdim, float inv_tau, float q_scale, cudaStream_t stream) {
    // few requests: narrow tiles, so that more CTAs share the work
    const int want = (num_requests * H * ((vdim * DS + 127) / 128) < 148) ? 32 : 128;
    const int threads = min(want, (vdim * DS + 31) / 32 * 32);
    const int cols = threads / DS;
    dim3 grid((vdim + cols - 1) / cols, H, num_requests);
    const size_t smem = (size_t)kGlaTokens * (3 * R * DS + cols) * sizeof(float);
    static size_t have = 0;
    ensure_dynamic_smem(gla_scan_kernel<T, R, DS>, smem, have);
    gla_scan_kernel<T, R, DS><<<grid, threads, smem, stream>>>((const T*)q, (const T*)k, (const T*)v, row_stride, z, o, state, cu,
                                                               start_pos, slots, request_list, H, dim, vdim, inv_tau, q_scale);
    return launch_status();
}

// q, k: [tokens, H*dim] and v: [tokens, H*vdim], column views of one projection buffer (common row stride, in
// elements); z: float32 [tokens, H*dim]; o: float32 [tokens, H*vdim]; state: float32 [slots, H, dim, vdim].
extern "C" int lb_gla_scan(const void* q, const void* k, const void* v, long row_stride, const float* z, float* o, float* state,
                           const int* cu, const int* start_pos, const int* slots, const int* request_list, int num_requests,
                           int H, int dim, int vdim, float tau, float q_scale, int dtype, void* stream) {
    if (num_requests <= 0) return kOk;
    if (H <= 0 || dim <= 0 || vdim <= 0 || !(tau > 0.f)) return kBadSize;
    if (dim > 512) return kTooLarge;
    cudaStream_t st = (cudaStream_t)stream;
#define LB_GLA(R_, DS_) LB_DISPATCH_DTYPE(dtype, return (launch_gla_scan<T, R_, DS_>(q, k, v, row_stride, z, o, state, cu, start_pos, \
        slots, request_list, num_requests, H, dim, vdim, 1.f / tau, q_scale, st)))
    if (dim <= 16) { LB_GLA(16, 1); }
    else if (dim <= 32) { LB_GLA(32, 1); }
    else if (dim <= 64) { LB_GLA(64, 1); }
    else if (dim <= 128) { LB_GLA(64, 2); }
    else if (dim <= 256) { LB_GLA(64, 4); }
    else { LB_GLA(64, 8); }
#undef LB_GLA
    return kOk;
}

// grid (rows, heads)
template <typename T>
__global__ void gla_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, long gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, int H, int vdim, float eps) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int h = blockIdx.y;
    const float* orow = o + (row * H + h) * vdim;
    float ss = 0.f;
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) ss += orow[c] * orow[c];
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        const float g = to_f32(gate[row * gate_stride + h * vdim + c]);
        out[(row * H + h) * vdim + c] = from_f32<T>(orow[c] * inv * weight[c] * silu_f(g));
    }
}

extern "C" int lb_gla_norm_gate(const float* o, const void* gate, long gate_stride, const float* weight, void* out, int rows,
                                int H, int vdim, float eps, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || vdim <= 0) return kBadSize;
    const int threads = min(256, (vdim + 31) / 32 * 32);
    dim3 grid(rows, H);
    LB_DISPATCH_DTYPE(dtype, gla_norm_gate_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        o, (const T*)gate, gate_stride, weight, (T*)out, H, vdim, eps));
    return launch_status();
}

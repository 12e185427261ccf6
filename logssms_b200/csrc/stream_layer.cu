// Pre-norm layers on a residual stream that is kept in 32-bit whatever the activation dtype.
//
//   embed_norm      : x[t] = N(table[id_t]) * w                     (the stream's first value; table rows are activations)
//   stream_add_norm : v = x + s * y   (s: a scale per channel, or none; without y: v = x)
//                     x_out = v (may be x itself), h = N(v) * w rounded to the activation dtype (what the next
//                     sublayer's products read)
//   stream_side     : v = x + s * y as above, then the token's side input
//                       a = gelu_tanh(G v) * e      (G [dim, H]; e: `dim` columns of the token's row of a side table)
//                       u = P a                     (P [H, dim])
//                       v <- v + u / sqrt(mean(u^2) + eps) * w_side
//                     x_out = v, and, when a norm follows at once, h = N(v) * w_next
//
// N is a layer norm without bias ((v - mean) / sqrt(var + eps), var the mean of the squared deviations, both passes
// over the row held in shared memory) or an RMS norm.  Sums, norms and the stream are float32; G, P and the tables
// are read in the dtype they are held in and multiplied in float32.
#include "lb200/common.cuh"
using namespace lb200;

enum : int { kLayerNorm = 0, kRmsNorm = 1 };

// 1 / sqrt(var + eps) and the mean of the row in shared memory (`row`, H floats); all threads get both
__device__ __forceinline__ void row_stats(const float* row, int H, int kind, float eps, float* red, float& mean, float& inv) {
    mean = 0.f;
    if (kind == kLayerNorm) {
        float s = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) s += row[c];
        mean = block_sum(s, red) / (float)H;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float d = row[c] - mean;
        ss += d * d;
    }
    inv = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps);
}

template <typename T>
__global__ void embed_norm_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                  const float* __restrict__ w, float eps, int H, int V, int kind, int* bad_ids) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && bad_ids) atomicAdd(bad_ids, 1);
        id = min(max(id, 0), V - 1);
    }
    const T* src = table + (size_t)id * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) row[c] = to_f32(src[c]);
    __syncthreads();
    float mean, inv;
    row_stats(row, H, kind, eps, red, mean, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[t * H + c] = (row[c] - mean) * inv * w[c];
}

extern "C" int lb_embed_norm(float* out, const void* table, const int* ids, const float* w, float eps, int tokens, int H, int V,
                             int kind, int* bad_ids, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || V <= 0 || (size_t)H * sizeof(float) > 160 * 1024 || (kind != kLayerNorm && kind != kRmsNorm)) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(embed_norm_kernel<T>, smem, have);
        embed_norm_kernel<T><<<tokens, threads, smem, (cudaStream_t)stream>>>(out, (const T*)table, ids, w, eps, H, V, kind, bad_ids);
    });
    return launch_status();
}

template <typename T>
__global__ void stream_add_norm_kernel(const float* x, const T* __restrict__ y, const float* __restrict__ ls,
                                       const float* __restrict__ w, float eps, float* x_out, T* __restrict__ h_out, int H, int kind) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[base + c];
        if (y != nullptr) v += (ls != nullptr ? ls[c] : 1.f) * to_f32(y[base + c]);
        row[c] = v;
        if (x_out != nullptr) x_out[base + c] = v;
    }
    if (h_out == nullptr) return;
    __syncthreads();
    float mean, inv;
    row_stats(row, H, kind, eps, red, mean, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) h_out[base + c] = from_f32<T>((row[c] - mean) * inv * w[c]);
}

extern "C" int lb_stream_add_norm(const float* x, const void* y, const float* ls, const float* w, float eps, float* x_out,
                                  void* h_out, int rows, int H, int kind, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    if (H <= 0 || (size_t)H * sizeof(float) > 160 * 1024 || (kind != kLayerNorm && kind != kRmsNorm)) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (size_t)H * sizeof(float);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(stream_add_norm_kernel<T>, smem, have);
        stream_add_norm_kernel<T><<<rows, threads, smem, (cudaStream_t)stream>>>(x, (const T*)y, ls, w, eps, x_out, (T*)h_out, H, kind);
    });
    return launch_status();
}

// grid (tokens); shared memory: row [H] | u [H] | a [dim]
template <typename T>
__global__ void stream_side_kernel(const float* x, const T* __restrict__ y, const float* __restrict__ ls,
                                   const int* __restrict__ ids, const T* __restrict__ side_table, int table_width, int offset,
                                   int V, const T* __restrict__ gate_w, const T* __restrict__ proj_w,
                                   const float* __restrict__ side_w, float side_eps, int dim, const float* __restrict__ next_w,
                                   float next_eps, int next_kind, float* x_out, T* __restrict__ h_out, int H) {
    extern __shared__ float smem[];
    __shared__ float red[32];
    float* row = smem;
    float* u = smem + H;
    float* a = smem + 2 * H;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const size_t t = blockIdx.x, base = t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[base + c];
        if (y != nullptr) v += (ls != nullptr ? ls[c] : 1.f) * to_f32(y[base + c]);
        row[c] = v;
    }
    __syncthreads();
    const int id = min(max(ids[t], 0), V - 1);
    const T* e = side_table + (size_t)id * table_width + offset;
    for (int d = warp; d < dim; d += nwarps) {
        const T* g = gate_w + (size_t)d * H;
        float acc = 0.f;
        for (int c = lane; c < H; c += 32) acc += to_f32(g[c]) * row[c];
        acc = warp_sum(acc);
        if (lane == 0)
            a[d] = 0.5f * acc * (1.f + tanhf(0.7978845608028654f * (acc + 0.044715f * acc * acc * acc))) * to_f32(e[d]);
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const T* p = proj_w + (size_t)c * dim;
        float acc = 0.f;
        for (int d = 0; d < dim; ++d) acc += to_f32(p[d]) * a[d];
        u[c] = acc;
        ss += acc * acc;
    }
    const float inv_u = 1.f / sqrtf(block_sum(ss, red) / (float)H + side_eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = row[c] + u[c] * inv_u * side_w[c];
        row[c] = v;
        x_out[base + c] = v;
    }
    if (h_out == nullptr) return;
    __syncthreads();
    float mean, inv;
    row_stats(row, H, next_kind, next_eps, red, mean, inv);
    for (int c = threadIdx.x; c < H; c += blockDim.x) h_out[base + c] = from_f32<T>((row[c] - mean) * inv * next_w[c]);
}

extern "C" int lb_stream_side(const float* x, const void* y, const float* ls, const int* ids, const void* side_table,
                              int table_width, int offset, int V, const void* gate_w, const void* proj_w, const float* side_w,
                              float side_eps, int dim, const float* next_w, float next_eps, int next_kind, float* x_out,
                              void* h_out, int rows, int H, int dtype, void* stream) {
    if (rows <= 0) return kOk;
    const size_t smem = ((size_t)2 * H + dim) * sizeof(float);
    if (H <= 0 || dim <= 0 || offset < 0 || offset + dim > table_width || V <= 0 || smem > 200 * 1024) return kBadSize;
    if (h_out != nullptr && next_kind != kLayerNorm && next_kind != kRmsNorm) return kBadSize;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(stream_side_kernel<T>, smem, have);
        stream_side_kernel<T><<<rows, threads, smem, (cudaStream_t)stream>>>(
            x, (const T*)y, ls, ids, (const T*)side_table, table_width, offset, V, (const T*)gate_w, (const T*)proj_w, side_w,
            side_eps, dim, next_w, next_eps, next_kind, x_out, (T*)h_out, H);
    });
    return launch_status();
}

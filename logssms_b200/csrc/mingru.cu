// minGRU: a gated recurrence per channel whose gates read the current token only.
//
//   z = sigmoid(pz + bz),  u = px + bx,  c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0)
//   S_t = (1 - z_t) S_{t-1} + z_t c_t,   out_t = S_t * silu(pg)
//
// `proj` [tokens, 3 * width] holds the three input products pz | px | pg of a token side by side (activation dtype);
// the biases, the gates, the candidate and the state are float32.  The state of a request lives in its slot
// [slots, width]; a request that starts at position 0 starts from zeros whatever the slot holds.
//
//   mingru_scan          : a thread per (request, channel) walks the request's tokens: decoded tokens, short portions,
//                          everything in a float32 engine
//   mingru_chunk_reduce, : long portions in chunks of `kChunk` tokens side by side: every chunk first folds its tokens
//   mingru_chunk_scan      into (A, B) with S_end = A S_begin + B; then every chunk folds the (A, B) of the chunks
//                          before it in its request into its own S_begin and walks its tokens once more
#include "lb200/common.cuh"
using namespace lb200;

constexpr int kThreads = 128;
constexpr int kChunk = 64;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// one token of one channel: S <- (1 - z) S + z c; returns S * silu(g)
__device__ __forceinline__ float mingru_token(float& S, float pz, float px, float pg, float bz, float bx) {
    const float z = sigmoid_f(pz + bz);
    const float u = px + bx;
    const float c = u >= 0.f ? u + 0.5f : sigmoid_f(u);
    S = (1.f - z) * S + z * c;
    return S * silu_f(pg);
}

// grid (ceil(width / kThreads), requests or listed requests)
template <typename T>
__global__ void __launch_bounds__(kThreads) mingru_scan_kernel(
        const T* __restrict__ proj, long row_stride, const float* __restrict__ bias_z, const float* __restrict__ bias_x,
        float* __restrict__ state, const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
        const int* __restrict__ request_list, T* __restrict__ out, int W) {
    const int b = request_list != nullptr ? request_list[blockIdx.y] : blockIdx.y;
    const int c = blockIdx.x * kThreads + threadIdx.x;
    if (b < 0 || c >= W) return;
    const int t0 = cu[b], t1 = cu[b + 1];
    float* slot = state + (size_t)slots[b] * W;
    float S = start_pos[b] > 0 ? slot[c] : 0.f;
    const float bz = bias_z[c], bx = bias_x[c];
    int t = t0;
    for (; t + 4 <= t1; t += 4) {           // four tokens' loads in flight
        float pz[4], px[4], pg[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const T* row = proj + (size_t)(t + k) * row_stride;
            pz[k] = to_f32(row[c]); px[k] = to_f32(row[W + c]); pg[k] = to_f32(row[2 * W + c]);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) out[(size_t)(t + k) * W + c] = from_f32<T>(mingru_token(S, pz[k], px[k], pg[k], bz, bx));
    }
    for (; t < t1; ++t) {
        const T* row = proj + (size_t)t * row_stride;
        out[(size_t)t * W + c] = from_f32<T>(mingru_token(S, to_f32(row[c]), to_f32(row[W + c]), to_f32(row[2 * W + c]), bz, bx));
    }
    if (t1 > t0) slot[c] = S;
}

extern "C" int lb_mingru_scan(const void* proj, long row_stride, const float* bias_z, const float* bias_x, float* state,
                              const int* cu, const int* start_pos, const int* slots, const int* request_list, void* out,
                              int num_requests, int W, int dtype, void* stream) {
    if (num_requests <= 0) return kOk;
    if (W <= 0 || num_requests > 65535) return kBadSize;
    dim3 grid((W + kThreads - 1) / kThreads, num_requests);
    LB_DISPATCH_DTYPE(dtype, mingru_scan_kernel<T><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        (const T*)proj, row_stride, bias_z, bias_x, state, cu, start_pos, slots, request_list, (T*)out, W));
    return launch_status();
}

// grid (ceil(width / kThreads), chunks); chunks: int32 [n, 2] (request, first token of the chunk within its portion), request -1: no work
template <typename T>
__global__ void __launch_bounds__(kThreads) mingru_chunk_reduce_kernel(
        const T* __restrict__ proj, long row_stride, const float* __restrict__ bias_z, const float* __restrict__ bias_x,
        const int* __restrict__ cu, const int* __restrict__ chunks, float* __restrict__ fold_a, float* __restrict__ fold_b, int W) {
    const int i = blockIdx.y, b = chunks[2 * i];
    const int c = blockIdx.x * kThreads + threadIdx.x;
    if (b < 0 || c >= W) return;
    const int t0 = cu[b] + chunks[2 * i + 1], t1 = min(t0 + kChunk, cu[b + 1]);
    const float bz = bias_z[c], bx = bias_x[c];
    float A = 1.f, B = 0.f;
    for (int t = t0; t < t1; ++t) {
        const T* row = proj + (size_t)t * row_stride;
        const float z = sigmoid_f(to_f32(row[c]) + bz);
        const float u = to_f32(row[W + c]) + bx;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        A *= 1.f - z;
        B = (1.f - z) * B + z * cand;
    }
    fold_a[(size_t)i * W + c] = A;
    fold_b[(size_t)i * W + c] = B;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) mingru_chunk_scan_kernel(
        const T* __restrict__ proj, long row_stride, const float* __restrict__ bias_z, const float* __restrict__ bias_x,
        float* state, const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
        const int* __restrict__ chunks, const float* __restrict__ fold_a, const float* __restrict__ fold_b,
        float* __restrict__ new_state, T* __restrict__ out, int W) {
    const int i = blockIdx.y, b = chunks[2 * i];
    const int c = blockIdx.x * kThreads + threadIdx.x;
    if (b < 0 || c >= W) return;
    const int off = chunks[2 * i + 1];
    const int t0 = cu[b] + off, t1 = min(t0 + kChunk, cu[b + 1]);
    float S = start_pos[b] > 0 ? state[(size_t)slots[b] * W + c] : 0.f;
    for (int j = i - off / kChunk; j < i; ++j) S = fold_a[(size_t)j * W + c] * S + fold_b[(size_t)j * W + c];
    const float bz = bias_z[c], bx = bias_x[c];
    for (int t = t0; t < t1; ++t) {
        const T* row = proj + (size_t)t * row_stride;
        out[(size_t)t * W + c] = from_f32<T>(mingru_token(S, to_f32(row[c]), to_f32(row[W + c]), to_f32(row[2 * W + c]), bz, bx));
    }
    // the slot is read by every chunk of the request: the last chunk leaves the new state beside it, and
    // `mingru_state_store` moves it there when all chunks are done
    if (t1 == cu[b + 1]) new_state[(size_t)b * W + c] = S;
}

// grid (ceil(width / kThreads), listed long requests)
__global__ void __launch_bounds__(kThreads) mingru_state_store_kernel(float* __restrict__ state, const float* __restrict__ new_state,
                                                                      const int* __restrict__ slots, const int* __restrict__ per_request, int W) {
    const int b = per_request[3 * blockIdx.y];
    const int c = blockIdx.x * kThreads + threadIdx.x;
    if (b < 0 || c >= W) return;
    state[(size_t)slots[b] * W + c] = new_state[(size_t)b * W + c];
}

extern "C" int lb_mingru_chunked(const void* proj, long row_stride, const float* bias_z, const float* bias_x, float* state,
                                 const int* cu, const int* start_pos, const int* slots, const int* chunks, int num_chunks,
                                 const int* per_request, int num_long, float* fold_a, float* fold_b, float* new_state, void* out,
                                 int W, int dtype, void* stream) {
    if (num_chunks <= 0 || num_long <= 0) return kOk;
    if (W <= 0 || num_chunks > 65535 || num_long > 65535) return kBadSize;
    dim3 grid((W + kThreads - 1) / kThreads, num_chunks);
    dim3 grid_req((W + kThreads - 1) / kThreads, num_long);
    LB_DISPATCH_DTYPE(dtype, {
        mingru_chunk_reduce_kernel<T><<<grid, kThreads, 0, (cudaStream_t)stream>>>((const T*)proj, row_stride, bias_z, bias_x, cu, chunks,
                                                                                  fold_a, fold_b, W);
        mingru_chunk_scan_kernel<T><<<grid, kThreads, 0, (cudaStream_t)stream>>>((const T*)proj, row_stride, bias_z, bias_x, state, cu,
                                                                                start_pos, slots, chunks, fold_a, fold_b, new_state,
                                                                                (T*)out, W);
        mingru_state_store_kernel<<<grid_req, kThreads, 0, (cudaStream_t)stream>>>(state, new_state, slots, per_request, W);
    });
    return launch_status();
}

extern "C" int lb_mingru_chunk() { return kChunk; }

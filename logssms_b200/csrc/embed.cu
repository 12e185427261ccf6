// Embedding row gather fused with the embedding multiplier.
//   out[t, :] = round(table[ids[t], :] * multiplier)
// Replaces the reference's gather kernel (csrc/jit/index.cu) plus the separate multiply of
// python/logssms/models/falcon_h1.py:213.  Ids outside [0, vocab) are clamped and counted in
// `bad_ids` (a device int the host may read); they never index out of the table.
#include "lb200/common.cuh"
using namespace lb200;

template <typename T>
__global__ void embed_gather_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                    int H, int V, float mult, int* bad_ids) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && bad_ids) atomicAdd(bad_ids, 1);
        id = min(max(id, 0), V - 1);
    }
    const T* src = table + (size_t)id * H;
    T* dst = out + (size_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = from_f32<T>(to_f32(src[c]) * mult);
}

// Row gather without scaling: out[i, :] = src[rows[i], :] (used to pick the positions whose logits are wanted).
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ src, const int* __restrict__ rows, int H) {
    pdl_trigger();
    const T* s = src + (size_t)rows[blockIdx.x] * H;
    T* d = out + (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) d[c] = s[c];
}

extern "C" int lb_embed_gather(void* out, const void* table, const int* ids, int T_, int H, int V, float mult,
                               int* bad_ids, int dtype, void* stream) {
    if (T_ <= 0) return kOk;
    if (H <= 0 || V <= 0) return kBadSize;
    const int threads = H >= 1024 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, embed_gather_kernel<T><<<T_, threads, 0, (cudaStream_t)stream>>>(
        (T*)out, (const T*)table, ids, H, V, mult, bad_ids));
    return launch_status();
}

extern "C" int lb_gather_rows(void* out, const void* src, const int* rows, int n, int H, int dtype, void* stream) {
    if (n <= 0) return kOk;
    const int threads = H >= 1024 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, gather_rows_kernel<T><<<n, threads, 0, (cudaStream_t)stream>>>(
        (T*)out, (const T*)src, rows, H));
    return launch_status();
}

// Token embedding plus a hashed embedding of the (previous token, token) pair, summed in 32-bit:
//   out[t, :] = table[id_t, :] * scale + pairs[row_t, :]
//   row_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets,  or row `buckets` for a sequence's first token.
// The token before a portion's first one is the request's state `prev_state[slot]` (int32 per slot); the block of a
// portion's first token reads it and then stores the portion's last id there, so a request's state is touched by
// one block only.  `out_act` (may be null) is the sum rounded to the activation dtype.
template <typename T>
__global__ void embed_pair_kernel(float* __restrict__ out_f32, T* __restrict__ out_act, const T* __restrict__ table,
                                  const T* __restrict__ pairs, const int* __restrict__ ids, const int* __restrict__ token_req,
                                  const int* __restrict__ cu, const int* __restrict__ start_pos, const int* __restrict__ slots,
                                  int* prev_state, int H, int V, int buckets, long long mul_prev, long long mul_cur,
                                  float scale, int* bad_ids) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && bad_ids) atomicAdd(bad_ids, 1);
        id = min(max(id, 0), V - 1);
    }
    const int b = token_req[t];
    const int first = cu[b];
    int prev;
    if (t > first) {
        prev = min(max(ids[t - 1], 0), V - 1);
    } else {
        prev = start_pos[b] > 0 ? prev_state[slots[b]] : -1;
        __syncthreads();                               // every thread has read the state before it is replaced
        if (threadIdx.x == 0) prev_state[slots[b]] = min(max(ids[cu[b + 1] - 1], 0), V - 1);
    }
    const long long row = prev < 0 ? (long long)buckets : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    const T* src = table + (size_t)id * H;
    const T* pr = pairs + (size_t)row * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float v = to_f32(src[c]) * scale + to_f32(pr[c]);
        out_f32[(size_t)t * H + c] = v;
        if (out_act != nullptr) out_act[(size_t)t * H + c] = from_f32<T>(v);
    }
}

extern "C" int lb_embed_pair(float* out_f32, void* out_act, const void* table, const void* pairs, const int* ids,
                             const int* token_req, const int* cu, const int* start_pos, const int* slots, int* prev_state,
                             int T_, int H, int V, int buckets, long long mul_prev, long long mul_cur, float scale,
                             int* bad_ids, int dtype, void* stream) {
    if (T_ <= 0) return kOk;
    if (H <= 0 || V <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return kBadSize;
    const int threads = H >= 1024 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, embed_pair_kernel<T><<<T_, threads, 0, (cudaStream_t)stream>>>(
        out_f32, (T*)out_act, (const T*)table, (const T*)pairs, ids, token_req, cu, start_pos, slots, prev_state, H, V,
        buckets, mul_prev, mul_cur, scale, bad_ids));
    return launch_status();
}

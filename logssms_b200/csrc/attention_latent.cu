// Attention over a cache of latents (one compressed row per token, shared by all heads) with a rotated key part.
//
// Per token the cache keeps c [rank] (the normalised latent) and kr [rot] (one rotated key part for all heads).
// A head's key is [W_uk,h c | kr] and its value W_uv,h c.  The kernels work in the latent space: the query's
// unrotated part is folded through W_uk,h first (qa = W_uk,h^T q, `lb_heads_matmul`), scores are
// (qa . c + q_rot . kr) * scale, the weighted sum of the c rows is expanded through W_uv,h afterwards.
//
//  latent_prepare   : per token: RMSNorm of the first `rank` columns of the down-projection -> cache "c";
//                     rotation of its last `rot` columns -> cache "kr"; rotation of every head's query part, in place
//  heads_matmul     : out[t, h, n] = sum_k a[t, h, k] * w[h, k, n]     (32-bit accumulation)
//  latent_attention : softmax attention of listed tokens over their request's pages, keys j with
//                     0 <= p - j < window (window 0: all earlier keys).  One warp per (token, head); the warps of a
//                     CTA are heads of one token and share its key tiles in shared memory; scores, softmax weights
//                     and the weighted sum are 32-bit.
#include "lb200/common.cuh"
using namespace lb200;

// grid (tokens); the rotation pairs column i with i + rd/2 among the first rd columns of a rotated part
template <typename T>
__global__ void latent_prepare_kernel(T* proj, long row_stride, int q_cols, int H, int nope, int rot, int rank,
                                      const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                      const float* __restrict__ cos_sin, int table_rows, int rd,
                                      const float* __restrict__ norm_w, float eps, T* __restrict__ c_cache,
                                      T* __restrict__ kr_cache, int write_cache) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    T* row = proj + t * row_stride;
    const int pos = min(max(positions[t], 0), table_rows - 1);
    const float* cs = cos_sin + (size_t)pos * rd;
    const int half = rd >> 1;
    const size_t slot = (size_t)slot_mapping[t];
    // latent: RMSNorm in 32-bit
    const T* d = row + q_cols;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(d[i]); ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
    if (write_cache) {
        for (int i = threadIdx.x; i < rank; i += blockDim.x) c_cache[slot * rank + i] = from_f32<T>(to_f32(d[i]) * inv * norm_w[i]);
        // the shared rotated key part
        const T* kr = d + rank;
        for (int i = threadIdx.x; i < rot; i += blockDim.x) {
            float v = to_f32(kr[i]);
            if (i < half) v = v * cs[i] - to_f32(kr[i + half]) * cs[half + i];
            else if (i < rd) v = v * cs[i - half] + to_f32(kr[i - half]) * cs[i];
            kr_cache[slot * rot + i] = from_f32<T>(v);
        }
    }
    // every head's rotated query part, in place (a thread owns a pair)
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        T* qr = row + (size_t)h * (nope + rot) + nope;
        const float u = to_f32(qr[j]), w = to_f32(qr[j + half]);
        qr[j] = from_f32<T>(u * cs[j] - w * cs[half + j]);
        qr[j + half] = from_f32<T>(w * cs[j] + u * cs[half + j]);
    }
}

extern "C" int lb_latent_prepare(void* proj, long row_stride, int q_cols, int H, int nope, int rot, int rank,
                                 const int* positions, const int* slot_mapping, const float* cos_sin, int table_rows, int rd,
                                 const float* norm_w, float eps, void* c_cache, void* kr_cache, int write_cache, int tokens,
                                 int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || nope < 0 || rot < 0 || rank <= 0 || rd < 0 || rd > rot || (rd & 1)) return kBadSize;
    LB_DISPATCH_DTYPE(dtype, latent_prepare_kernel<T><<<tokens, 128, 0, (cudaStream_t)stream>>>(
        (T*)proj, row_stride, q_cols, H, nope, rot, rank, positions, slot_mapping, cos_sin, table_rows, rd, norm_w, eps,
        (T*)c_cache, (T*)kr_cache, write_cache));
    return launch_status();
}

// grid (ceil(N / 128), H, ceil(tokens / 8)); a[t*a_row + h*a_head + k]; w [H, K, N]; out[t*o_row + h*o_head + n]
constexpr int kHmTokens = 8;
template <typename T>
__global__ void heads_matmul_kernel(const T* __restrict__ a, long a_row, long a_head, const T* __restrict__ w,
                                    T* __restrict__ out, long o_row, long o_head, int tokens, int K, int N) {
    extern __shared__ float as[];                    // [kHmTokens][K]
    const int h = blockIdx.y, t0 = blockIdx.z * kHmTokens;
    const int nt = min(kHmTokens, tokens - t0);
    for (int i = threadIdx.x; i < kHmTokens * K; i += blockDim.x) {
        const int tt = i / K, kk = i % K;
        as[i] = tt < nt ? to_f32(a[(size_t)(t0 + tt) * a_row + (size_t)h * a_head + kk]) : 0.f;
    }
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float acc[kHmTokens];
#pragma unroll
    for (int tt = 0; tt < kHmTokens; ++tt) acc[tt] = 0.f;
    const T* wp = w + (size_t)h * K * N + n;
    for (int kk = 0; kk < K; ++kk) {
        const float wv = to_f32(wp[(size_t)kk * N]);
#pragma unroll
        for (int tt = 0; tt < kHmTokens; ++tt) acc[tt] += as[tt * K + kk] * wv;
    }
    for (int tt = 0; tt < nt; ++tt) out[(size_t)(t0 + tt) * o_row + (size_t)h * o_head + n] = from_f32<T>(acc[tt]);
}

extern "C" int lb_heads_matmul(const void* a, long a_row, long a_head, const void* w, void* out, long o_row, long o_head,
                               int tokens, int H, int K, int N, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (H <= 0 || K <= 0 || N <= 0) return kBadSize;
    const size_t smem = (size_t)kHmTokens * K * sizeof(float);
    if (smem > 160 * 1024) return kTooLarge;
    dim3 grid((N + 127) / 128, H, (tokens + kHmTokens - 1) / kHmTokens);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(heads_matmul_kernel<T>, smem, have);
        heads_matmul_kernel<T><<<grid, 128, smem, (cudaStream_t)stream>>>((const T*)a, a_row, a_head, (const T*)w, (T*)out,
                                                                         o_row, o_head, tokens, K, N);
    });
    return launch_status();
}

constexpr int kLaWarps = 4;       // heads of one token per CTA
constexpr int kLaTile = 32;       // keys per tile: one per lane
constexpr int kLaMaxPieces = 16;  // rank <= 32 * 16

// grid (listed tokens, ceil(H / kLaWarps))
template <typename T>
__global__ void __launch_bounds__(kLaWarps * 32) latent_attention_kernel(
        const T* __restrict__ qa, const T* __restrict__ q_rot, long q_rot_row, long q_rot_head,
        const T* __restrict__ c_cache, const T* __restrict__ kr_cache, const int* __restrict__ block_table, int table_width,
        const int* __restrict__ token_req, const int* __restrict__ positions, const int* __restrict__ token_list,
        T* __restrict__ out, int H, int rank, int rot, int page_size, float scale, int window) {
    extern __shared__ float sm[];
    const int D = rank + rot, DP = D + 1;
    float* qs = sm;                        // [kLaWarps][D]
    float* ks = sm + kLaWarps * D;         // [kLaTile][DP]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = token_list ? token_list[blockIdx.x] : blockIdx.x;
    if (t < 0) return;
    const int h = blockIdx.y * kLaWarps + warp;
    const bool live = h < H;
    const int p = positions[t];
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    if (live) {
        for (int d = lane; d < D; d += 32)
            qs[warp * D + d] = scale * (d < rank ? to_f32(qa[((size_t)t * H + h) * rank + d])
                                                 : to_f32(q_rot[(size_t)t * q_rot_row + (size_t)h * q_rot_head + d - rank]));
    }
    const int pieces = (rank + 31) >> 5;
    float acc[kLaMaxPieces];
#pragma unroll
    for (int i = 0; i < kLaMaxPieces; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int j0 = lo; j0 <= p; j0 += kLaTile) {
        const int nvalid = min(kLaTile, p - j0 + 1);
        __syncthreads();
        for (int jj = warp; jj < nvalid; jj += kLaWarps) {
            const int j = j0 + jj;
            const size_t off = (size_t)pages[j / page_size] * page_size + j % page_size;
            for (int d = lane; d < D; d += 32)
                ks[jj * DP + d] = d < rank ? to_f32(c_cache[off * rank + d]) : to_f32(kr_cache[off * rot + d - rank]);
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < nvalid) {
            s = 0.f;
            const float* kr = ks + lane * DP;
            const float* qr = qs + warp * D;
            for (int d = 0; d < D; ++d) s += qr[d] * kr[d];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);           // m = -inf at the first tile: 0
        const float pj = lane < nvalid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < kLaMaxPieces; ++i) acc[i] *= corr;
        for (int jj = 0; jj < nvalid; ++jj) {
            const float pp = __shfl_sync(0xffffffffu, pj, jj);
            const float* kr = ks + jj * DP;
#pragma unroll
            for (int i = 0; i < kLaMaxPieces; ++i)
                if (i < pieces) { const int r = lane + 32 * i; if (r < rank) acc[i] += pp * kr[r]; }
        }
        m = m_new;
    }
    if (!live) return;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kLaMaxPieces; ++i)
        if (i < pieces) { const int r = lane + 32 * i; if (r < rank) out[((size_t)t * H + h) * rank + r] = from_f32<T>(acc[i] * inv); }
}

// qa: [tokens, H, rank]; q_rot: the rotated query parts inside another buffer (row and head strides in elements);
// caches: [pages, page_size, rank] and [pages, page_size, rot]; out: [tokens, H, rank] (listed rows only)
extern "C" int lb_latent_attention(const void* qa, const void* q_rot, long q_rot_row, long q_rot_head, const void* c_cache,
                                   const void* kr_cache, const int* block_table, int table_width, const int* token_req,
                                   const int* positions, const int* token_list, int num_listed, void* out, int H, int rank,
                                   int rot, int page_size, float scale, int window, int dtype, void* stream) {
    if (num_listed <= 0) return kOk;
    if (H <= 0 || rank <= 0 || rot < 0 || page_size <= 0 || window < 0) return kBadSize;
    if (rank > 32 * kLaMaxPieces) return kTooLarge;
    const int D = rank + rot;
    const size_t smem = ((size_t)kLaWarps * D + (size_t)kLaTile * (D + 1)) * sizeof(float);
    if (smem > 200 * 1024) return kTooLarge;
    dim3 grid(num_listed, (H + kLaWarps - 1) / kLaWarps);
    LB_DISPATCH_DTYPE(dtype, {
        static size_t have = 0;
        ensure_dynamic_smem(latent_attention_kernel<T>, smem, have);
        latent_attention_kernel<T><<<grid, kLaWarps * 32, smem, (cudaStream_t)stream>>>(
            (const T*)qa, (const T*)q_rot, q_rot_row, q_rot_head, (const T*)c_cache, (const T*)kr_cache, block_table,
            table_width, token_req, positions, token_list, (T*)out, H, rank, rot, page_size, scale, window);
    });
    return launch_status();
}

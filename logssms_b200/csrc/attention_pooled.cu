// Grouped-query attention over a sliding window of tokens plus pooled blocks behind it, with rotated values.
//
//   Query i sees the tokens j with 0 <= i - j < window and, as ONE key and value each, every block b of `pool` tokens
//   (positions b*pool .. b*pool + pool - 1) that lies wholly behind the window: b*pool + pool - 1 <= i - window, i.e.
//   the first floor((i - window + 1) / pool) blocks.  A block's key and value are the means of its tokens' cached keys
//   and values.  Tokens that have left the window and whose block is not yet complete behind it are not seen.  Tokens
//   and blocks share one softmax.
//
//   Queries and keys are rotated over neighbouring pairs (columns 2i, 2i + 1 of the first `rot` columns, angle
//   p * f_i); values are rotated the same way over ALL their columns by their own position and cached so; the
//   weighted sum of the values of query i is turned back by -i.  cos/sin come from tables [positions, n] (cos of
//   the n/2 pairs, then sin) in float32.
//
//   pooled_prepare : per (token, head): rotate the query; rotate key and value and store them at the token's slot
//   pooled_blocks  : per token that ends a block: the means of the block's cached keys and values, stored at the
//                    block's entry of a second paged cache (one entry per `pool` tokens)
//   pooled_attention      : a warp per (token, head); a lane scores one key at a time, the lanes share the value
//                           columns; scores, softmax and sums in float32 (every dtype, every size, every step)
//   pooled_attention_tile : a CTA per (run of up to 16 neighbouring tokens of a request, kv head): the keys the run's
//                           queries see are staged through shared memory once for all queries of the group
#include "lb200/common.cuh"
using namespace lb200;

// grid (tokens, Hq + 2 * Hkv)
template <typename T>
__global__ void pooled_prepare_kernel(const T* __restrict__ qkv, long row_stride, const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping, const float* __restrict__ qk_table, int rot,
                                      const float* __restrict__ v_table, int v_rot, int table_rows, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int dim, int vdim,
                                      int write_kv) {
    const size_t t = blockIdx.x;
    int head = blockIdx.y;
    const int pos = min(max(positions[t], 0), table_rows - 1);
    const T* src;
    T* dst;
    const float* cs;
    int n, r;
    if (head < Hq) {
        src = qkv + t * row_stride + (size_t)head * dim;
        dst = q_out + (t * Hq + head) * dim;
        n = dim; r = rot; cs = qk_table + (size_t)pos * rot;
    } else {
        if (!write_kv) return;
        const long slot = slot_mapping[t];
        if (slot < 0) return;
        head -= Hq;
        if (head < Hkv) {
            src = qkv + t * row_stride + (size_t)Hq * dim + (size_t)head * dim;
            dst = k_cache + ((size_t)slot * Hkv + head) * dim;
            n = dim; r = rot; cs = qk_table + (size_t)pos * rot;
        } else {
            head -= Hkv;
            src = qkv + t * row_stride + (size_t)(Hq + Hkv) * dim + (size_t)head * vdim;
            dst = v_cache + ((size_t)slot * Hkv + head) * vdim;
            n = vdim; r = v_rot; cs = v_table + (size_t)pos * v_rot;
        }
    }
    const int half = r >> 1;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        float val = to_f32(src[c]);
        if (c < r) {
            const float partner = to_f32(src[c ^ 1]);
            const float co = cs[c >> 1], si = cs[half + (c >> 1)];
            val = (c & 1) ? val * co + partner * si : val * co - partner * si;
        }
        dst[c] = from_f32<T>(val);
    }
}

extern "C" int lb_pooled_prepare(const void* qkv, long row_stride, const int* positions, const int* slot_mapping,
                                 const float* qk_table, int rot, const float* v_table, int v_rot, int table_rows, void* q_out,
                                 void* k_cache, void* v_cache, int tokens, int Hq, int Hkv, int dim, int vdim, int write_kv,
                                 int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || dim <= 0 || vdim <= 0 || rot < 0 || rot > dim || (rot & 1) || v_rot < 0 || v_rot > vdim || (v_rot & 1)
        || Hq + 2 * Hkv > 65535 || table_rows <= 0)
        return kBadSize;
    dim3 grid(tokens, Hq + 2 * Hkv);
    const int threads = max(dim, vdim) > 64 ? 128 : 64;
    LB_DISPATCH_DTYPE(dtype, pooled_prepare_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)qkv, row_stride, positions, slot_mapping, qk_table, rot, v_table, v_rot, table_rows, (T*)q_out, (T*)k_cache,
        (T*)v_cache, Hq, Hkv, dim, vdim, write_kv));
    return launch_status();
}

// grid (tokens, Hkv): the token that ends a block writes the block's means
template <typename T>
__global__ void pooled_blocks_kernel(const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ kp_cache,
                                     T* __restrict__ vp_cache, const int* __restrict__ positions, const int* __restrict__ token_req,
                                     const int* __restrict__ block_table, int table_width, const int* __restrict__ pooled_slots,
                                     int Hkv, int dim, int vdim, int page_size, int pool) {
    const int t = blockIdx.x, g = blockIdx.y;
    const int pos = positions[t];
    if (pos < 0 || (pos + 1) % pool != 0) return;
    const long out_slot = pooled_slots[t];
    if (out_slot < 0) return;
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int first = pos + 1 - pool;
    const float inv = 1.f / (float)pool;
    for (int c = threadIdx.x; c < dim + vdim; c += blockDim.x) {
        float sum = 0.f;
        for (int j = first; j <= pos; ++j) {
            const int page = pages[j / page_size];
            if (page < 0) continue;
            const size_t slot = (size_t)page * page_size + j % page_size;
            sum += c < dim ? to_f32(k_cache[(slot * Hkv + g) * dim + c]) : to_f32(v_cache[(slot * Hkv + g) * vdim + (c - dim)]);
        }
        if (c < dim) kp_cache[((size_t)out_slot * Hkv + g) * dim + c] = from_f32<T>(sum * inv);
        else vp_cache[((size_t)out_slot * Hkv + g) * vdim + (c - dim)] = from_f32<T>(sum * inv);
    }
}

extern "C" int lb_pooled_blocks(const void* k_cache, const void* v_cache, void* kp_cache, void* vp_cache, const int* positions,
                                const int* token_req, const int* block_table, int table_width, const int* pooled_slots,
                                int tokens, int Hkv, int dim, int vdim, int page_size, int pool, int dtype, void* stream) {
    if (tokens <= 0) return kOk;
    if (Hkv <= 0 || Hkv > 65535 || dim <= 0 || vdim <= 0 || page_size <= 0 || pool <= 0) return kBadSize;
    dim3 grid(tokens, Hkv);
    const int threads = dim + vdim > 128 ? 256 : 128;
    LB_DISPATCH_DTYPE(dtype, pooled_blocks_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const T*)k_cache, (const T*)v_cache, (T*)kp_cache, (T*)vp_cache, positions, token_req, block_table, table_width,
        pooled_slots, Hkv, dim, vdim, page_size, pool));
    return launch_status();
}

// ------------------------------------------------------------------------------------------------ attention, a warp per row
constexpr int kWarps = 4;            // (token, head) rows of a CTA: neighbouring heads of one token
constexpr int kMaxValueRegs = 8;     // value columns per lane: vdim <= 256

// the cache row of key number `kk` of a query: the first `blocks` keys are pooled blocks, the others the window's tokens
__device__ __forceinline__ long key_row(int kk, int blocks, int first, const int* __restrict__ pages, const int* __restrict__ pooled_pages,
                                        int page_size, bool& pooled) {
    pooled = kk < blocks;
    const int e = pooled ? kk : first + (kk - blocks);
    const int page = (pooled ? pooled_pages : pages)[e / page_size];
    return page < 0 ? -1 : (long)page * page_size + e % page_size;
}

// grid (tokens, ceil(Hq / kWarps)); dynamic shared memory: kWarps * dim floats (the scaled queries)
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) pooled_attention_kernel(
        const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, const T* __restrict__ kp_cache,
        const T* __restrict__ vp_cache, const int* __restrict__ block_table, int table_width, const int* __restrict__ pooled_table,
        int pooled_width, const int* __restrict__ token_req, const int* __restrict__ positions, const int* __restrict__ token_list,
        const float* __restrict__ v_table, int v_rot, int table_rows, T* __restrict__ out, int Hq, int Hkv, int dim, int vdim,
        int page_size, float scale, int window, int pool) {
    extern __shared__ float q_s[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = token_list != nullptr ? token_list[blockIdx.x] : blockIdx.x;
    const int head = blockIdx.y * kWarps + warp;
    if (t < 0 || head >= Hq) return;
    const int g = head / (Hq / Hkv);
    const int pos = positions[t];
    float* qs = q_s + warp * dim;
    for (int c = lane; c < dim; c += 32) qs[c] = to_f32(q[((size_t)t * Hq + head) * dim + c]) * scale;
    __syncwarp();
    const int* pages = block_table + (size_t)token_req[t] * table_width;
    const int* pooled_pages = pooled_table + (size_t)token_req[t] * pooled_width;
    const int first = max(0, pos - window + 1);
    const int blocks = max(0, (pos - window + 1) / pool);
    const int keys = blocks + (pos - first + 1);
    float m = -INFINITY, l = 0.f, acc[kMaxValueRegs];
#pragma unroll
    for (int r = 0; r < kMaxValueRegs; ++r) acc[r] = 0.f;
    for (int k0 = 0; k0 < keys; k0 += 32) {
        const int kk = k0 + lane;
        float s = -INFINITY;
        long row = -1;
        bool pooled = false;
        if (kk < keys) {
            row = key_row(kk, blocks, first, pages, pooled_pages, page_size, pooled);
            if (row >= 0) {
                const T* kr = (pooled ? kp_cache : k_cache) + ((size_t)row * Hkv + g) * dim;
                float a0 = 0.f, a1 = 0.f;
                int c = 0;
                for (; c + 2 <= dim; c += 2) { a0 += qs[c] * to_f32(kr[c]); a1 += qs[c + 1] * to_f32(kr[c + 1]); }
                if (c < dim) a0 += qs[c] * to_f32(kr[c]);
                s = a0 + a1;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
        const float p = s == -INFINITY ? 0.f : expf(s - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < kMaxValueRegs; ++r) acc[r] *= corr;
        const int n = min(32, keys - k0);
        for (int j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long rj = __shfl_sync(0xffffffffu, row, j);
            const bool pooled_j = (k0 + j) < blocks;
            if (rj < 0 || pj == 0.f) continue;
            const T* vr = (pooled_j ? vp_cache : v_cache) + ((size_t)rj * Hkv + g) * vdim;
#pragma unroll
            for (int r = 0; r < kMaxValueRegs; ++r) {
                const int c = lane + 32 * r;
                if (c < vdim) acc[r] += pj * to_f32(vr[c]);
            }
        }
    }
    // the summed values, turned back by the query's position (pairs of neighbouring columns: neighbouring lanes)
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    const float* cs = v_table + (size_t)min(max(pos, 0), table_rows - 1) * v_rot;
    const int half = v_rot >> 1;
#pragma unroll
    for (int r = 0; r < kMaxValueRegs; ++r) {
        const int c = lane + 32 * r;
        const float own = acc[r] * inv_l;
        const float partner = __shfl_xor_sync(0xffffffffu, own, 1);
        if (c < vdim) {
            float val = own;
            if (c < v_rot) {
                const float co = cs[c >> 1], si = cs[half + (c >> 1)];
                val = (c & 1) ? own * co - partner * si : own * co + partner * si;
            }
            out[((size_t)t * Hq + head) * vdim + c] = from_f32<T>(val);
        }
    }
}

extern "C" int lb_pooled_attention(const void* q, const void* k_cache, const void* v_cache, const void* kp_cache,
                                   const void* vp_cache, const int* block_table, int table_width, const int* pooled_table,
                                   int pooled_width, const int* token_req, const int* positions, const int* token_list,
                                   int num_tokens, const float* v_table, int v_rot, int table_rows, void* out, int Hq, int Hkv,
                                   int dim, int vdim, int page_size, float scale, int window, int pool, int dtype, void* stream) {
    if (num_tokens <= 0) return kOk;
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || dim <= 0 || vdim <= 0 || page_size <= 0 || window <= 0 || pool <= 0 || (v_rot & 1)
        || v_rot > vdim || table_rows <= 0)
        return kBadSize;
    if (vdim > 32 * kMaxValueRegs || (size_t)kWarps * dim * sizeof(float) > 48 * 1024) return kTooLarge;
    dim3 grid(num_tokens, (Hq + kWarps - 1) / kWarps);
    LB_DISPATCH_DTYPE(dtype, pooled_attention_kernel<T><<<grid, kWarps * 32, (size_t)kWarps * dim * sizeof(float), (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (const T*)kp_cache, (const T*)vp_cache, block_table, table_width,
        pooled_table, pooled_width, token_req, positions, token_list, v_table, v_rot, table_rows, (T*)out, Hq, Hkv, dim, vdim,
        page_size, scale, window, pool));
    return launch_status();
}

// Softmax attention over the paged cache with the options that the plain kernels do not have:
//
//   * value heads of another width than query/key heads;
//   * a window that also keeps the first tokens of the sequence: the query at position p sees key j
//     when j <= p and (p - j < window or j < keep_first); window 0 keeps every key;
//   * a distance bias taken off the score: s = (q . k) * scale - r1[h] * ln(1 + r2[h] * (p - j));
//   * mixing of the heads' weights after the softmax: w'_h = sum_g talk[h][g] * w_g, head h then reads
//     the values of its own KV head with w'_h.
//
// One warp per (token, query head).  Keys are visited in tiles of 32 whose boundaries are multiples of 32
// in absolute position, first the kept tokens that lie behind the window, then the window, so the
// arithmetic of a query depends on its own position only (the same bits however the prompt was cut
// and whatever else is in the batch).
//
// Mixing after the softmax needs every head's normalised weights over all keys.  Instead of keeping them,
// head g's warp applies its weights to the values of EVERY KV head c: A[g][c] = sum_j w_g(j) v_c(j).
// The mixed output of head h is then sum_g talk[h][g] * A[g][kv(h)], which a second small kernel forms.
// The weights themselves are never stored and one pass over the keys suffices.
#include "common.cuh"

#include <algorithm>

struct BiasedArgs {
    const void* q;           // [tokens][heads][dim]
    const void* k_pages;     // [pages][kv_heads][page_size][dim]
    const void* v_pages;     // [pages][kv_heads][page_size][vdim]
    const int* block_table;  // [entries][table_width]
    const int* entry_of_token;
    const int* positions;
    const float* r1;  // [heads] or null: no distance bias
    const float* r2;
    void* out;        // spread == 1: float32 [tokens][heads][kv_heads][vdim]; else [tokens][heads][vdim] of T
    float scale;
    int tokens, heads, kv_heads, dim, vdim, page_size, table_width, window, keep_first;
    int spread;  // 1: every KV head's values (for mixing); 0: the head's own
};

constexpr int BIASED_WARPS = 4;

template <typename T, int NACC>
__global__ void __launch_bounds__(BIASED_WARPS * 32) biased_attention_kernel(BiasedArgs a) {
    extern __shared__ float q_staged[];  // [BIASED_WARPS][dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = static_cast<long long>(blockIdx.x) * BIASED_WARPS + warp;
    if (item >= static_cast<long long>(a.tokens) * a.heads) return;
    const int token = static_cast<int>(item / a.heads), head = static_cast<int>(item % a.heads);
    const int d = a.dim, vd = a.vdim;
    const int vchunks = (vd + 31) / 32;
    pdl_trigger();
    const float r1 = a.r1 ? a.r1[head] : 0.0f, r2 = a.r1 ? a.r2[head] : 0.0f;
    pdl_wait();
    const int own_kv = head / (a.heads / a.kv_heads);
    const int first_value_head = a.spread ? 0 : own_kv;
    const int value_heads = a.spread ? a.kv_heads : 1;
    const int position = a.positions[token];
    const int* table = a.block_table + static_cast<size_t>(a.entry_of_token[token]) * a.table_width;
    const T* k_pages = static_cast<const T*>(a.k_pages);
    const T* v_pages = static_cast<const T*>(a.v_pages);

    float* q = q_staged + warp * d;
    const T* q_src = static_cast<const T*>(a.q) + (static_cast<size_t>(token) * a.heads + head) * d;
    for (int i = lane; i < d; i += 32) q[i] = to_float(q_src[i]);
    __syncwarp();

    const int lowest = a.window > 0 ? max(position - a.window + 1, 0) : 0;
    const int kept_end = a.window > 0 ? min(a.keep_first, lowest) : 0;  // keys [0, kept_end) lie behind the window and stay
    float running_max = -INFINITY, denom = 0.0f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;

    // Two runs of tiles: the kept first tokens, then the window.
    for (int run = 0; run < 2; ++run) {
        const int from = run == 0 ? 0 : lowest, to = run == 0 ? kept_end - 1 : position;  // inclusive
        for (int tile = (from / 32) * 32; tile <= to; tile += 32) {
            const int key = tile + lane;
            const bool valid = key >= from && key <= to;
            long long slot = -1;  // page * page_size + offset of this lane's key, -1 when masked
            if (valid) {
                const int page = table[key / a.page_size];
                if (page >= 0) slot = static_cast<long long>(page) * a.page_size + key % a.page_size;
            }
            float score = -INFINITY;
            if (slot >= 0) {
                const long long page = slot / a.page_size, offset = slot % a.page_size;
                const T* k_row = k_pages + ((page * a.kv_heads + own_kv) * a.page_size + offset) * d;
                float dot = 0.0f;
                for (int i = 0; i < d; ++i) dot = fmaf(q[i], to_float(k_row[i]), dot);
                score = dot * a.scale;
                if (a.r1) score -= r1 * logf(1.0f + r2 * static_cast<float>(position - key));
            }
            const float new_max = fmaxf(running_max, warp_max(score));
            if (new_max == -INFINITY) continue;  // nothing visible yet (uniform across the warp)
            const float p = slot >= 0 ? expf(score - new_max) : 0.0f;
            const float rescale = expf(running_max - new_max);  // 0 on the first tile (exp(-inf))
            denom = denom * rescale + warp_sum(p);
            running_max = new_max;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] *= rescale;
            for (int j = 0; j < 32; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                const long long sj = __shfl_sync(0xffffffffu, slot, j);
                if (sj < 0) continue;  // uniform across the warp
                const long long page = sj / a.page_size, offset = sj % a.page_size;
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const int c = i / vchunks, e = lane + 32 * (i % vchunks);
                    if (c < value_heads && e < vd) {
                        const T* v_row = v_pages + ((page * a.kv_heads + first_value_head + c) * a.page_size + offset) * vd;
                        acc[i] = fmaf(pj, to_float(v_row[e]), acc[i]);
                    }
                }
            }
        }
    }
    const float inv = 1.0f / denom;
    if (a.spread) {
        float* out = static_cast<float*>(a.out) + (static_cast<size_t>(token) * a.heads + head) * a.kv_heads * vd;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int c = i / vchunks, e = lane + 32 * (i % vchunks);
            if (c < value_heads && e < vd) out[c * vd + e] = acc[i] * inv;
        }
    } else {
        T* out = static_cast<T*>(a.out) + (static_cast<size_t>(token) * a.heads + head) * vd;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int e = lane + 32 * i;
            if (i < vchunks && e < vd) out[e] = from_float<T>(acc[i] * inv);
        }
    }
}

template <typename T>
static int launch_biased(const BiasedArgs& a, cudaStream_t stream) {
    const int per_lane = (a.spread ? a.kv_heads : 1) * ((a.vdim + 31) / 32);
    const long long items = static_cast<long long>(a.tokens) * a.heads;
    const int blocks = static_cast<int>((items + BIASED_WARPS - 1) / BIASED_WARPS);
    const size_t smem = static_cast<size_t>(BIASED_WARPS) * a.dim * sizeof(float);
    if (per_lane <= 2) return launch_kernel(biased_attention_kernel<T, 2>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 4) return launch_kernel(biased_attention_kernel<T, 4>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 8) return launch_kernel(biased_attention_kernel<T, 8>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 16) return launch_kernel(biased_attention_kernel<T, 16>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 32) return launch_kernel(biased_attention_kernel<T, 32>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 64) return launch_kernel(biased_attention_kernel<T, 64>, blocks, BIASED_WARPS * 32, smem, stream, a);
    return ME_ERR_UNSUPPORTED;
}

ME_EXPORT int me_biased_attention(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                  const int* entry_of_token, const int* positions, const float* r1, const float* r2,
                                  void* out, int type, float scale, int tokens, int heads, int kv_heads, int dim,
                                  int vdim, int page_size, int table_width, int window, int keep_first, int spread,
                                  cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads % kv_heads || dim < 1 || vdim < 1 || dim > 2048) return ME_ERR_UNSUPPORTED;
    if ((r1 == nullptr) != (r2 == nullptr) || window < 0 || keep_first < 0) return ME_ERR_ARGUMENT;
    BiasedArgs a{q, k_pages, v_pages, block_table, entry_of_token, positions, r1, r2, out, scale,
                 tokens, heads, kv_heads, dim, vdim, page_size, table_width, window, keep_first, spread};
    return type == ME_BF16 ? launch_biased<__nv_bfloat16>(a, stream) : launch_biased<float>(a, stream);
}

// out[t][h][e] = sum_g talk[h][g] * spread[t][g][kv(h)][e], ascending g.
template <typename T>
__global__ void mix_heads_kernel(const float* __restrict__ spread, const float* __restrict__ talk, T* __restrict__ out,
                                 int tokens, int heads, int kv_heads, int vdim) {
    pdl_trigger();
    pdl_wait();
    const size_t total = static_cast<size_t>(tokens) * heads * vdim;
    const int group = heads / kv_heads;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int e = static_cast<int>(idx % vdim);
        const int h = static_cast<int>((idx / vdim) % heads);
        const size_t t = idx / (static_cast<size_t>(vdim) * heads);
        const float* row = spread + t * heads * kv_heads * vdim + static_cast<size_t>(h / group) * vdim + e;
        float sum = 0.0f;
        for (int g = 0; g < heads; ++g) sum = fmaf(talk[h * heads + g], row[static_cast<size_t>(g) * kv_heads * vdim], sum);
        out[idx] = from_float<T>(sum);
    }
}

ME_EXPORT int me_mix_heads(const float* spread, const float* talk, void* out, int type, int tokens, int heads,
                           int kv_heads, int vdim, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * heads * vdim;
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
    if (type == ME_BF16)
        return launch_kernel(mix_heads_kernel<__nv_bfloat16>, blocks, threads, 0, stream, spread, talk,
                             static_cast<__nv_bfloat16*>(out), tokens, heads, kv_heads, vdim);
    return launch_kernel(mix_heads_kernel<float>, blocks, threads, 0, stream, spread, talk, static_cast<float*>(out),
                         tokens, heads, kv_heads, vdim);
}

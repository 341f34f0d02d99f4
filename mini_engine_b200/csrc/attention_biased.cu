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

// ---- the same with 16-byte loads: head widths that are multiples of 8 (bfloat16) or 4 (float32)

template <typename T>
struct Packed;
template <>
struct Packed<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
    }
};
template <>
struct Packed<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 x = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // a bfloat16 is the upper half of a float
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// One block of VEC_WARPS warps per (token, query head): 4 in float32 always (the same bits for a token in a
// prompt and decoded alone), in bfloat16 1 when the step has items enough to fill the GPU and 16 when it has few.  Warp w takes the key tiles whose number (absolute
// position / 32) is w modulo VEC_WARPS, keeps its own running maximum, denominator and sums, and warp 0 adds
// the warps' results in ascending order: which warp visits which tile, and the order of every sum, depend on
// the query's position only.  A lane owns NV segments of N consecutive value elements among the (value
// heads x vdim) values of a key: segment u = lane + 32 * i is elements (u % per_row) * N .. of value head
// u / per_row.  Values are fetched for four keys at a time, all loads ahead of the arithmetic.
template <typename T, int NV, int VEC_WARPS>
__global__ void __launch_bounds__(VEC_WARPS * 32) biased_attention_vec_kernel(BiasedArgs a) {
    constexpr int N = Packed<T>::N;
    extern __shared__ __align__(16) float vec_shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x / a.heads, head = blockIdx.x % a.heads;
    const int d = a.dim, vd = a.vdim;
    float* q = vec_shared;                                  // [dim]
    float* part_stat = q + ((d + 3) / 4) * 4;               // [VEC_WARPS][2] maximum, denominator
    float* part_acc = part_stat + VEC_WARPS * 2;            // [VEC_WARPS][NV][N][32]
    pdl_trigger();
    const float r1 = a.r1 ? a.r1[head] : 0.0f, r2 = a.r1 ? a.r2[head] : 0.0f;
    pdl_wait();
    const int own_kv = head / (a.heads / a.kv_heads);
    const int first_value_head = a.spread ? 0 : own_kv;
    const int value_heads = a.spread ? a.kv_heads : 1;
    const int per_row = vd / N, segments = value_heads * per_row;
    long long segment_offset[NV];  // where the lane's segments lie behind a key's first value head
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int u = lane + 32 * i;
        segment_offset[i] = u < segments ? (static_cast<long long>(first_value_head + u / per_row) * a.page_size) * vd + (u % per_row) * N : -1;
    }
    const int position = a.positions[token];
    const int* table = a.block_table + static_cast<size_t>(a.entry_of_token[token]) * a.table_width;
    const T* k_pages = static_cast<const T*>(a.k_pages);
    const T* v_pages = static_cast<const T*>(a.v_pages);

    const T* q_src = static_cast<const T*>(a.q) + (static_cast<size_t>(token) * a.heads + head) * d;
    for (int i = threadIdx.x; i < d; i += VEC_WARPS * 32) q[i] = to_float(q_src[i]);
    __syncthreads();

    const int lowest = a.window > 0 ? max(position - a.window + 1, 0) : 0;
    const int kept_end = a.window > 0 ? min(a.keep_first, lowest) : 0;
    float running_max = -INFINITY, denom = 0.0f;
    float acc[NV][N];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < N; ++e) acc[i][e] = 0.0f;

    for (int run = 0; run < 2; ++run) {
        const int from = run == 0 ? 0 : lowest, to = run == 0 ? kept_end - 1 : position;  // inclusive
        for (int tile = (from / 32) * 32; tile <= to; tile += 32) {
            if ((tile >> 5) % VEC_WARPS != warp) continue;
            const int key = tile + lane;
            const bool valid = key >= from && key <= to;
            int page = -1, offset = 0;
            if (valid) {
                page = table[key / a.page_size];
                offset = key % a.page_size;
            }
            float score = -INFINITY;
            if (page >= 0) {
                const T* k_row = k_pages + ((static_cast<long long>(page) * a.kv_heads + own_kv) * a.page_size + offset) * d;
                float dot = 0.0f;
#pragma unroll 4
                for (int i = 0; i < d; i += N) {
                    float k[N];
                    Packed<T>::load(k_row + i, k);
#pragma unroll
                    for (int e = 0; e < N; ++e) dot = fmaf(q[i + e], k[e], dot);
                }
                score = dot * a.scale;
                if (a.r1) score -= r1 * logf(1.0f + r2 * static_cast<float>(position - key));
            }
            const float new_max = fmaxf(running_max, warp_max(score));
            if (new_max == -INFINITY) continue;  // nothing visible in this tile (uniform across the warp)
            const float p = page >= 0 ? expf(score - new_max) : 0.0f;
            const float rescale = expf(running_max - new_max);  // 0 on the warp's first tile (exp(-inf))
            denom = denom * rescale + warp_sum(p);
            running_max = new_max;
#pragma unroll
            for (int i = 0; i < NV; ++i)
#pragma unroll
                for (int e = 0; e < N; ++e) acc[i][e] *= rescale;
            // element offset of the key's value row in value head 0, -1 when masked
            const long long row = page >= 0 ? (static_cast<long long>(page) * a.kv_heads * a.page_size + offset) * vd : -1;
            // Values: for KEYS keys at a time, all loads ahead of the arithmetic.  One warp per item (a step
            // with items enough to fill every SM) takes one key at a time: fewer registers, more warps per SM.
            constexpr int KEYS = VEC_WARPS == 1 ? 1 : 4;
#pragma unroll 4
            for (int j0 = 0; j0 < 32; j0 += KEYS) {
                float pj[KEYS];
                long long rj[KEYS];
                float v[KEYS][NV][N];
#pragma unroll
                for (int u = 0; u < KEYS; ++u) {
                    pj[u] = __shfl_sync(0xffffffffu, p, j0 + u);
                    rj[u] = __shfl_sync(0xffffffffu, row, j0 + u);
                }
#pragma unroll
                for (int u = 0; u < KEYS; ++u)
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        if (rj[u] >= 0 && segment_offset[i] >= 0) {
                            Packed<T>::load(v_pages + rj[u] + segment_offset[i], v[u][i]);
                        } else {
#pragma unroll
                            for (int e = 0; e < N; ++e) v[u][i][e] = 0.0f;  // a masked key has weight 0 as well
                        }
                    }
#pragma unroll
                for (int u = 0; u < KEYS; ++u)
#pragma unroll
                    for (int i = 0; i < NV; ++i)
#pragma unroll
                        for (int e = 0; e < N; ++e) acc[i][e] = fmaf(pj[u], v[u][i][e], acc[i][e]);
            }
        }
    }
    // The warps' partial results meet in shared memory; warp 0 adds them in ascending order.
    if (lane == 0) {
        part_stat[warp * 2] = running_max;
        part_stat[warp * 2 + 1] = denom;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < N; ++e) part_acc[((warp * NV + i) * N + e) * 32 + lane] = acc[i][e];
    __syncthreads();
    if (warp != 0) return;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < VEC_WARPS; ++w) top = fmaxf(top, part_stat[w * 2]);
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < N; ++e) acc[i][e] = 0.0f;
#pragma unroll
    for (int w = 0; w < VEC_WARPS; ++w) {
        const float m = part_stat[w * 2];
        if (m == -INFINITY) continue;  // this warp saw no key
        const float factor = expf(m - top);
        total = fmaf(part_stat[w * 2 + 1], factor, total);
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int e = 0; e < N; ++e) acc[i][e] = fmaf(part_acc[((w * NV + i) * N + e) * 32 + lane], factor, acc[i][e]);
    }
    const float inv = 1.0f / total;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int u = lane + 32 * i;
        if (u >= segments) continue;
        const int c = u / per_row, e0 = (u % per_row) * N;
        if (a.spread) {
            float* out = static_cast<float*>(a.out) + ((static_cast<size_t>(token) * a.heads + head) * a.kv_heads + c) * vd + e0;
#pragma unroll
            for (int e = 0; e < N; ++e) out[e] = acc[i][e] * inv;
        } else {
            T* out = static_cast<T*>(a.out) + (static_cast<size_t>(token) * a.heads + head) * vd + e0;
#pragma unroll
            for (int e = 0; e < N; ++e) out[e] = from_float<T>(acc[i][e] * inv);
        }
    }
}

template <typename T, int NV, int VEC_WARPS>
static int launch_biased_vec_with(const BiasedArgs& a, cudaStream_t stream) {
    static SharedMemoryOptIn opt_in;
    constexpr int N = Packed<T>::N;
    const size_t smem = (static_cast<size_t>((a.dim + 3) / 4) * 4 + VEC_WARPS * 2 + static_cast<size_t>(VEC_WARPS) * NV * N * 32) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        const int code = opt_in(biased_attention_vec_kernel<T, NV, VEC_WARPS>, static_cast<int>(smem));
        if (code) return code;
    }
    const long long items = static_cast<long long>(a.tokens) * a.heads;
    if (items > 0x7fffffffll) return ME_ERR_UNSUPPORTED;
    return launch_kernel_in_order(biased_attention_vec_kernel<T, NV, VEC_WARPS>, static_cast<int>(items), VEC_WARPS * 32, smem, stream, a);
}

constexpr long long ITEMS_THAT_FILL_THE_GPU = 2048;

template <typename T, int NV>
static int launch_biased_vec_as(const BiasedArgs& a, cudaStream_t stream) {
    if constexpr (sizeof(T) == 4) {
        return launch_biased_vec_with<T, NV, 4>(a, stream);
    } else {
        if (static_cast<long long>(a.tokens) * a.heads >= ITEMS_THAT_FILL_THE_GPU) return launch_biased_vec_with<T, NV, 1>(a, stream);
        return launch_biased_vec_with<T, NV, 16>(a, stream);
    }
}

template <typename T>
static int launch_biased_vec(const BiasedArgs& a, cudaStream_t stream, bool& taken) {
    constexpr int N = Packed<T>::N;
    const int segments = (a.spread ? a.kv_heads : 1) * (a.vdim / N);
    const int per_lane = (segments + 31) / 32;
    taken = true;
    if (per_lane <= 1) return launch_biased_vec_as<T, 1>(a, stream);
    if (per_lane <= 2) return launch_biased_vec_as<T, 2>(a, stream);
    if (per_lane <= 4) return launch_biased_vec_as<T, 4>(a, stream);
    if constexpr (N == 4) {
        if (per_lane <= 8) return launch_biased_vec_as<T, 8>(a, stream);
    }
    taken = false;
    return 0;
}

template <typename T>
static int launch_biased(const BiasedArgs& a, cudaStream_t stream) {
    // Which kernel runs depends on the model's sizes and the alignment of the engine's buffers only.
    constexpr int N = Packed<T>::N;
    const bool aligned = reinterpret_cast<uintptr_t>(a.k_pages) % 16 == 0 && reinterpret_cast<uintptr_t>(a.v_pages) % 16 == 0;
    if (a.dim % N == 0 && a.vdim % N == 0 && aligned) {
        bool taken = false;
        const int code = launch_biased_vec<T>(a, stream, taken);
        if (taken) return code;
    }
    const int per_lane = (a.spread ? a.kv_heads : 1) * ((a.vdim + 31) / 32);
    const long long items = static_cast<long long>(a.tokens) * a.heads;
    const int blocks = static_cast<int>((items + BIASED_WARPS - 1) / BIASED_WARPS);
    const size_t smem = static_cast<size_t>(BIASED_WARPS) * a.dim * sizeof(float);
    if (per_lane <= 2) return launch_kernel_in_order(biased_attention_kernel<T, 2>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 4) return launch_kernel_in_order(biased_attention_kernel<T, 4>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 8) return launch_kernel_in_order(biased_attention_kernel<T, 8>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 16) return launch_kernel_in_order(biased_attention_kernel<T, 16>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 32) return launch_kernel_in_order(biased_attention_kernel<T, 32>, blocks, BIASED_WARPS * 32, smem, stream, a);
    if (per_lane <= 64) return launch_kernel_in_order(biased_attention_kernel<T, 64>, blocks, BIASED_WARPS * 32, smem, stream, a);
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

// ------------------------------------------------------------- mixing in two kernels (fewer multiply-adds)
//
// The one-pass form above pays kv_heads times the value arithmetic for mixing after the softmax.  The form
// below keeps the scores instead: kernel 1 writes every (token, head)'s scores of its visible keys (32-bit,
// compacted: kept tokens first, then the window) and the softmax's maximum and denominator; kernel 2, one block
// per (token, KV head), turns the scores of ALL heads into normalised weights key by key, mixes them for the
// heads of its own group and applies the mixed weights to its values.  Per (token, key): heads x dim for the
// scores, heads x group for the mixing, group x vdim for the values, each once.  Tiles go to warps by tile
// number and partial results are added in ascending order, as above.

struct ScoreArgs {
    BiasedArgs a;
    float* scores;  // [tokens][heads][stride]
    float* stats;   // [tokens][heads][2] maximum, denominator
    int stride;     // most keys a query can see
};

template <typename T, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attention_scores_kernel(ScoreArgs s) {
    constexpr int N = Packed<T>::N;
    const BiasedArgs& a = s.a;
    extern __shared__ __align__(16) float score_shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x / a.heads, head = blockIdx.x % a.heads;
    const int d = a.dim;
    float* q = score_shared;                         // [dim]
    float* part_stat = q + ((d + 3) / 4) * 4;        // [WARPS][2]
    pdl_trigger();
    const float r1 = a.r1 ? a.r1[head] : 0.0f, r2 = a.r1 ? a.r2[head] : 0.0f;
    pdl_wait();
    const int own_kv = head / (a.heads / a.kv_heads);
    const int position = a.positions[token];
    const int* table = a.block_table + static_cast<size_t>(a.entry_of_token[token]) * a.table_width;
    const T* k_pages = static_cast<const T*>(a.k_pages);
    const T* q_src = static_cast<const T*>(a.q) + (static_cast<size_t>(token) * a.heads + head) * d;
    for (int i = threadIdx.x; i < d; i += WARPS * 32) q[i] = to_float(q_src[i]);
    __syncthreads();
    const bool packed = d % N == 0 && reinterpret_cast<uintptr_t>(a.k_pages) % 16 == 0;
    const int lowest = a.window > 0 ? max(position - a.window + 1, 0) : 0;
    const int kept_end = a.window > 0 ? min(a.keep_first, lowest) : 0;
    float* row = s.scores + (static_cast<size_t>(token) * a.heads + head) * s.stride;
    float running_max = -INFINITY, denom = 0.0f;
    for (int run = 0; run < 2; ++run) {
        const int from = run == 0 ? 0 : lowest, to = run == 0 ? kept_end - 1 : position;  // inclusive
        for (int tile = (from / 32) * 32; tile <= to; tile += 32) {
            if ((tile >> 5) % WARPS != warp) continue;
            const int key = tile + lane;
            const bool valid = key >= from && key <= to;
            int page = -1;
            if (valid) page = table[key / a.page_size];
            float score = -INFINITY;
            if (page >= 0) {
                const T* k_row = k_pages + ((static_cast<long long>(page) * a.kv_heads + own_kv) * a.page_size + key % a.page_size) * d;
                float dot = 0.0f;
                if (packed) {
#pragma unroll 4
                    for (int i = 0; i < d; i += N) {
                        float k[N];
                        Packed<T>::load(k_row + i, k);
#pragma unroll
                        for (int e = 0; e < N; ++e) dot = fmaf(q[i + e], k[e], dot);
                    }
                } else {
                    for (int i = 0; i < d; ++i) dot = fmaf(q[i], to_float(k_row[i]), dot);
                }
                score = dot * a.scale;
                if (a.r1) score -= r1 * logf(1.0f + r2 * static_cast<float>(position - key));
            }
            if (valid) row[run == 0 ? key : kept_end + (key - lowest)] = score;
            const float new_max = fmaxf(running_max, warp_max(score));
            if (new_max == -INFINITY) continue;
            const float p = page >= 0 ? expf(score - new_max) : 0.0f;
            denom = denom * expf(running_max - new_max) + warp_sum(p);
            running_max = new_max;
        }
    }
    if (lane == 0) {
        part_stat[warp * 2] = running_max;
        part_stat[warp * 2 + 1] = denom;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    float top = -INFINITY;
    for (int w = 0; w < WARPS; ++w) top = fmaxf(top, part_stat[w * 2]);
    float total = 0.0f;
    for (int w = 0; w < WARPS; ++w)
        if (part_stat[w * 2] != -INFINITY) total = fmaf(part_stat[w * 2 + 1], expf(part_stat[w * 2] - top), total);
    float* out = s.stats + (static_cast<size_t>(token) * a.heads + head) * 2;
    out[0] = top;
    out[1] = total;
}

constexpr int MIX_GROUP = 8;    // query heads per KV head, at most
constexpr int MIX_COLUMNS = 8;  // value elements per lane, at most: vdim <= 256

template <typename T, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attention_mix_values_kernel(ScoreArgs s, const float* __restrict__ talk) {
    const BiasedArgs& a = s.a;
    extern __shared__ __align__(16) float mix_shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x / a.kv_heads, kv = blockIdx.x % a.kv_heads;
    const int heads = a.heads, group = heads / a.kv_heads, vd = a.vdim;
    float* top = mix_shared;                 // [heads]
    float* inverse = top + heads;            // [heads] 1 / denominator
    float* mixing = inverse + heads;         // [group][heads] rows of the mixing matrix for this group's heads
    float* partial = mixing + group * heads; // [WARPS][group][vd]
    pdl_trigger();
    for (int i = threadIdx.x; i < group * heads; i += WARPS * 32) mixing[i] = talk[(kv * group + i / heads) * heads + i % heads];
    pdl_wait();
    for (int g = threadIdx.x; g < heads; g += WARPS * 32) {
        const float* st = s.stats + (static_cast<size_t>(token) * heads + g) * 2;
        top[g] = st[0];
        inverse[g] = 1.0f / st[1];
    }
    __syncthreads();
    const int position = a.positions[token];
    const int* table = a.block_table + static_cast<size_t>(a.entry_of_token[token]) * a.table_width;
    const T* v_pages = static_cast<const T*>(a.v_pages);
    const int lowest = a.window > 0 ? max(position - a.window + 1, 0) : 0;
    const int kept_end = a.window > 0 ? min(a.keep_first, lowest) : 0;
    const float* rows = s.scores + static_cast<size_t>(token) * heads * s.stride;
    float acc[MIX_GROUP][MIX_COLUMNS];
#pragma unroll
    for (int h = 0; h < MIX_GROUP; ++h)
#pragma unroll
        for (int i = 0; i < MIX_COLUMNS; ++i) acc[h][i] = 0.0f;
    for (int run = 0; run < 2; ++run) {
        const int from = run == 0 ? 0 : lowest, to = run == 0 ? kept_end - 1 : position;  // inclusive
        for (int tile = (from / 32) * 32; tile <= to; tile += 32) {
            if ((tile >> 5) % WARPS != warp) continue;
            const int key = tile + lane;
            const bool valid = key >= from && key <= to;
            long long value_row = -1;  // element offset of this key's values in this KV head
            float mixed[MIX_GROUP];
#pragma unroll
            for (int h = 0; h < MIX_GROUP; ++h) mixed[h] = 0.0f;
            if (valid) {
                const int page = table[key / a.page_size];
                if (page >= 0) {
                    value_row = ((static_cast<long long>(page) * a.kv_heads + kv) * a.page_size + key % a.page_size) * vd;
                    const int index = run == 0 ? key : kept_end + (key - lowest);
                    for (int g = 0; g < heads; ++g) {  // ascending g: the order of the mixed sum
                        const float w = expf(rows[static_cast<size_t>(g) * s.stride + index] - top[g]) * inverse[g];
#pragma unroll
                        for (int h = 0; h < MIX_GROUP; ++h)
                            if (h < group) mixed[h] = fmaf(mixing[h * heads + g], w, mixed[h]);
                    }
                }
            }
            for (int j = 0; j < 32; ++j) {
                const long long rj = __shfl_sync(0xffffffffu, value_row, j);
                float wj[MIX_GROUP];
#pragma unroll
                for (int h = 0; h < MIX_GROUP; ++h) wj[h] = __shfl_sync(0xffffffffu, mixed[h], j);
                if (rj < 0) continue;  // uniform across the warp
                const T* v_row = v_pages + rj;
#pragma unroll
                for (int i = 0; i < MIX_COLUMNS; ++i) {
                    const int e = lane + 32 * i;
                    if (e < vd) {
                        const float v = to_float(v_row[e]);
#pragma unroll
                        for (int h = 0; h < MIX_GROUP; ++h) acc[h][i] = fmaf(wj[h], v, acc[h][i]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < MIX_GROUP; ++h)
#pragma unroll
        for (int i = 0; i < MIX_COLUMNS; ++i) {
            const int e = lane + 32 * i;
            if (h < group && e < vd) partial[(warp * group + h) * vd + e] = acc[h][i];
        }
    __syncthreads();
    T* out = static_cast<T*>(a.out) + (static_cast<size_t>(token) * heads + kv * group) * vd;
    for (int i = threadIdx.x; i < group * vd; i += WARPS * 32) {
        float sum = 0.0f;
        for (int w = 0; w < WARPS; ++w) sum += partial[w * group * vd + i];
        out[i] = from_float<T>(sum);
    }
}

template <typename T, int WARPS>
static int launch_two_kernels(const ScoreArgs& s, const float* talk, cudaStream_t stream) {
    static SharedMemoryOptIn opt_in;
    const BiasedArgs& a = s.a;
    const int group = a.heads / a.kv_heads;
    const size_t smem1 = (static_cast<size_t>((a.dim + 3) / 4) * 4 + WARPS * 2) * sizeof(float);
    const size_t smem2 = (static_cast<size_t>(2) * a.heads + static_cast<size_t>(group) * a.heads + static_cast<size_t>(WARPS) * group * a.vdim) * sizeof(float);
    if (smem1 > 48 * 1024 || smem2 > 200 * 1024) return ME_ERR_UNSUPPORTED;
    if (smem2 > 48 * 1024) {
        const int code = opt_in(attention_mix_values_kernel<T, WARPS>, static_cast<int>(smem2));
        if (code) return code;
    }
    int code = launch_kernel_in_order(attention_scores_kernel<T, WARPS>, a.tokens * a.heads, WARPS * 32, smem1, stream, s);
    if (code) return code;
    return launch_kernel_in_order(attention_mix_values_kernel<T, WARPS>, a.tokens * a.kv_heads, WARPS * 32, smem2, stream, s, talk);
}

// Mixed attention in two kernels.  `scores` holds tokens * heads * stride floats, `stats` tokens * heads * 2;
// `stride` is the most keys a query of this step can see.  out: [tokens][heads][vdim] of the pages' type.
ME_EXPORT int me_mixed_attention(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                 const int* entry_of_token, const int* positions, const float* r1, const float* r2,
                                 const float* talk, float* scores, float* stats, int stride, void* out, int type,
                                 float scale, int tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                                 int table_width, int window, int keep_first, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads % kv_heads || heads / kv_heads > MIX_GROUP || vdim > 32 * MIX_COLUMNS || dim < 1 || vdim < 1) return ME_ERR_UNSUPPORTED;
    if ((r1 == nullptr) != (r2 == nullptr) || window < 0 || keep_first < 0 || talk == nullptr || stride < 1) return ME_ERR_ARGUMENT;
    if (static_cast<long long>(tokens) * heads > 0x7fffffffll) return ME_ERR_UNSUPPORTED;
    ScoreArgs s{{q, k_pages, v_pages, block_table, entry_of_token, positions, r1, r2, out, scale, tokens, heads,
                 kv_heads, dim, vdim, page_size, table_width, window, keep_first, 0},
                scores, stats, stride};
    // float32: four warps always (the same bits for a token in a prompt and decoded alone); bfloat16: two
    // warps when the step has blocks enough to fill the GPU, sixteen when it has few.
    if (type != ME_BF16) return launch_two_kernels<float, 4>(s, talk, stream);
    if (static_cast<long long>(tokens) * kv_heads >= 1024) return launch_two_kernels<__nv_bfloat16, 2>(s, talk, stream);
    return launch_two_kernels<__nv_bfloat16, 16>(s, talk, stream);
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

// Gated linear attention: a per-head matrix state with a decay per key channel.
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   S: [dim][vdim] per head, float32,
//   alpha_t = sigmoid(z_t)^(1/tau),  z_t = A2 (A1 h_t) + b  (a low-rank projection of the layer's input),
//
// then every head's o_t is divided by its root mean square over vdim (eps inside the root), multiplied by
// a weight [vdim] shared by the heads and by silu of a gate projection, and leaves in the compute dtype
// for the output projection.  The state of a request lives in its slot of the cache manager's state
// array between steps; an entry that starts at position 0 starts from zero.
//
// Scan kernel: one warp per (entry, head, 32 value columns).  Each lane owns one column of the state in
// registers ([dim] floats) and walks the entry's tokens in order; q, k and alpha of a chunk of tokens are
// prepared by the whole warp in shared memory first (the sum of the product's partial sums, the query
// scale, the decay from the low-rank sums in 32-bit), so the serial part is two multiply-adds per state
// element and token.  Columns are independent, hence the result does not depend on how the work is cut
// over warps, and a token's output depends on the tokens before it only through the state: the bits are
// the same for a whole prompt, its portions and single decoded tokens.
//
// Finish kernel: one warp per (token, head): unit norm, weight, gate.
#include "common.cuh"

#include <algorithm>

struct ScanArgs {
    const float* proj;  // [splits][tokens][width] partial sums of the fused input projection
    int splits;
    size_t split_stride;
    int width;                      // columns of a row of proj
    int q_col, k_col, v_col, a_col;  // first column of q [heads*dim], k [heads*dim], v [heads*vdim], low-rank [rank]
    const float* a2;       // [heads*dim][rank]
    const float* a2_bias;  // [heads*dim]
    const int* cu_tokens;   // [entries + 1]
    const int* state_slots; // [entries]
    const int* fresh;       // [entries] 1: the entry starts its request, the state starts at zero
    float* state;           // [slots + 1][heads][dim][vdim]
    float* out;             // [tokens][heads][vdim] float32: o_t before the norm
    float q_scale, inv_tau;
    int heads, dim, vdim, rank;
};

constexpr int SCAN_CHUNK = 16;

// log(sigmoid(z)) without overflow: -softplus(-z).
__device__ __forceinline__ float log_sigmoid(float z) {
    return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

template <int DIMP>  // dim rounded up: the registers a lane holds of its state column
__global__ void __launch_bounds__(32) gla_scan_kernel(ScanArgs a) {
    extern __shared__ float staged[];
    float* q_s = staged;                          // [SCAN_CHUNK][DIMP]
    float* k_s = q_s + SCAN_CHUNK * DIMP;         // [SCAN_CHUNK][DIMP]
    float* d_s = k_s + SCAN_CHUNK * DIMP;         // [SCAN_CHUNK][DIMP] decay
    float* v_s = d_s + SCAN_CHUNK * DIMP;         // [SCAN_CHUNK][32] this warp's value columns
    float* r_s = v_s + SCAN_CHUNK * 32;           // [SCAN_CHUNK][rank] low-rank sums
    const int entry = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int column = blockIdx.z * 32 + lane;
    const bool live = column < a.vdim;
    const int dim = a.dim;
    pdl_trigger();
    pdl_wait();
    const int begin = a.cu_tokens[entry], end = a.cu_tokens[entry + 1];
    float* state = a.state + ((static_cast<size_t>(a.state_slots[entry]) * a.heads + head) * dim) * a.vdim + column;

    float s[DIMP];
    const bool from_zero = a.fresh[entry] != 0;
#pragma unroll
    for (int d = 0; d < DIMP; ++d) s[d] = (live && !from_zero && d < dim) ? state[static_cast<size_t>(d) * a.vdim] : 0.0f;

    for (int chunk = begin; chunk < end; chunk += SCAN_CHUNK) {
        const int count = min(SCAN_CHUNK, end - chunk);
        __syncwarp();
        for (int i = lane; i < count * a.rank; i += 32) {
            const int t = i / a.rank, r = i % a.rank;
            const float* src = a.proj + static_cast<size_t>(chunk + t) * a.width + a.a_col + r;
            float sum = 0.0f;
            for (int p = 0; p < a.splits; ++p) sum += src[p * a.split_stride];
            r_s[t * a.rank + r] = sum;
        }
        __syncwarp();
        for (int i = lane; i < count * DIMP; i += 32) {
            const int t = i / DIMP, d = i % DIMP;
            float q = 0.0f, k = 0.0f, decay = 0.0f;
            if (d < dim) {
                const float* row = a.proj + static_cast<size_t>(chunk + t) * a.width + head * dim + d;
                for (int p = 0; p < a.splits; ++p) {
                    q += row[p * a.split_stride + a.q_col];
                    k += row[p * a.split_stride + a.k_col];
                }
                q *= a.q_scale;
                const float* w = a.a2 + static_cast<size_t>(head * dim + d) * a.rank;
                float z = 0.0f;
                for (int r = 0; r < a.rank; ++r) z = fmaf(w[r], r_s[t * a.rank + r], z);
                z += a.a2_bias[head * dim + d];
                decay = expf(log_sigmoid(z) * a.inv_tau);
            }
            q_s[i] = q, k_s[i] = k, d_s[i] = decay;
        }
        for (int t = 0; t < count; ++t) {
            float value = 0.0f;
            if (live) {
                const float* src = a.proj + static_cast<size_t>(chunk + t) * a.width + a.v_col + head * a.vdim + column;
                for (int p = 0; p < a.splits; ++p) value += src[p * a.split_stride];
            }
            v_s[t * 32 + lane] = value;
        }
        __syncwarp();
#pragma unroll 1
        for (int t = 0; t < count; ++t) {
            const float v = v_s[t * 32 + lane];
            const float4* q4 = reinterpret_cast<const float4*>(q_s + t * DIMP);
            const float4* k4 = reinterpret_cast<const float4*>(k_s + t * DIMP);
            const float4* d4 = reinterpret_cast<const float4*>(d_s + t * DIMP);
            float o = 0.0f;
#pragma unroll
            for (int d = 0; d < DIMP; d += 4) {
                const float4 qq = q4[d / 4], kk = k4[d / 4], dd = d4[d / 4];
                s[d + 0] = fmaf(dd.x, s[d + 0], kk.x * v);
                s[d + 1] = fmaf(dd.y, s[d + 1], kk.y * v);
                s[d + 2] = fmaf(dd.z, s[d + 2], kk.z * v);
                s[d + 3] = fmaf(dd.w, s[d + 3], kk.w * v);
                o = fmaf(s[d + 0], qq.x, o);
                o = fmaf(s[d + 1], qq.y, o);
                o = fmaf(s[d + 2], qq.z, o);
                o = fmaf(s[d + 3], qq.w, o);
            }
            if (live) a.out[(static_cast<size_t>(chunk + t) * a.heads + head) * a.vdim + column] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DIMP; ++d)
            if (d < dim) state[static_cast<size_t>(d) * a.vdim] = s[d];
    }
}

template <int DIMP>
static int launch_scan(const ScanArgs& a, int entries, cudaStream_t stream) {
    static SharedMemoryOptIn opt_in;
    const size_t smem = (static_cast<size_t>(SCAN_CHUNK) * (3 * DIMP + 32 + a.rank)) * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        const int code = opt_in(gla_scan_kernel<DIMP>, static_cast<int>(smem));
        if (code) return code;
    }
    const dim3 grid(entries, a.heads, (a.vdim + 31) / 32);
    return launch_kernel(gla_scan_kernel<DIMP>, grid, 32, smem, stream, a);
}

ME_EXPORT int me_gla_scan(const float* proj, int splits, long long split_stride, int width, int q_col, int k_col,
                          int v_col, int a_col, const float* a2, const float* a2_bias, const int* cu_tokens,
                          const int* state_slots, const int* fresh, float* state, float* out, float q_scale,
                          float tau, int entries, int heads, int dim, int vdim, int rank, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (dim < 1 || vdim < 1 || rank < 1 || heads < 1 || !(tau > 0.0f)) return ME_ERR_ARGUMENT;
    ScanArgs a{proj, splits, static_cast<size_t>(split_stride), width, q_col, k_col, v_col, a_col, a2, a2_bias,
               cu_tokens, state_slots, fresh, state, out, q_scale, 1.0f / tau, heads, dim, vdim, rank};
    if (dim <= 16) return launch_scan<16>(a, entries, stream);
    if (dim <= 32) return launch_scan<32>(a, entries, stream);
    if (dim <= 64) return launch_scan<64>(a, entries, stream);
    if (dim <= 128) return launch_scan<128>(a, entries, stream);
    if (dim <= 192) return launch_scan<192>(a, entries, stream);
    return ME_ERR_UNSUPPORTED;
}

// out[t][h][e] = weight[e] * o[t][h][e] * rsqrt(mean_e(o^2) + eps) * silu(gate[t][h][e]).
template <typename T>
__global__ void __launch_bounds__(128) gla_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj,
                                                         int splits, size_t split_stride, int width, int g_col,
                                                         const float* __restrict__ weight, float eps,
                                                         T* __restrict__ out, int tokens, int heads, int vdim) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = static_cast<long long>(blockIdx.x) * 4 + warp;
    pdl_trigger();
    pdl_wait();
    if (item >= static_cast<long long>(tokens) * heads) return;
    const size_t token = static_cast<size_t>(item / heads);
    const int head = static_cast<int>(item % heads);
    const float* row = o + (token * heads + head) * vdim;
    float sum_sq = 0.0f;
    for (int e = lane; e < vdim; e += 32) sum_sq = fmaf(row[e], row[e], sum_sq);
    sum_sq = warp_sum(sum_sq);
    const float inv = rsqrtf(sum_sq / static_cast<float>(vdim) + eps);
    const float* gate_row = proj + token * width + g_col + head * vdim;
    T* dst = out + (token * heads + head) * vdim;
    for (int e = lane; e < vdim; e += 32) {
        float gate = 0.0f;
        for (int p = 0; p < splits; ++p) gate += gate_row[p * split_stride + e];
        const float activated = gate / (1.0f + expf(-gate));
        dst[e] = from_float<T>(weight[e] * (row[e] * inv) * activated);
    }
}

ME_EXPORT int me_gla_finish(const float* o, const float* proj, int splits, long long split_stride, int width,
                            int g_col, const float* weight, float eps, void* out, int type, int tokens, int heads,
                            int vdim, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const long long items = static_cast<long long>(tokens) * heads;
    const int blocks = static_cast<int>((items + 3) / 4);
    if (type == ME_BF16)
        return launch_kernel(gla_finish_kernel<__nv_bfloat16>, blocks, 128, 0, stream, o, proj, splits,
                             (size_t)split_stride, width, g_col, weight, eps, static_cast<__nv_bfloat16*>(out), tokens,
                             heads, vdim);
    return launch_kernel(gla_finish_kernel<float>, blocks, 128, 0, stream, o, proj, splits, (size_t)split_stride, width,
                         g_col, weight, eps, static_cast<float*>(out), tokens, heads, vdim);
}

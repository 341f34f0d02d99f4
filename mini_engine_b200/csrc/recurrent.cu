// A gated linear recurrence per channel (the real-gated linear recurrent unit of Griffin-style blocks),
// over the flat batch of a step, from and into each request's state slot.
//
// The block's input projection arrives as float32 partial sums `proj [S][T][2 C]`: columns [0, C) are the gate
// branch, [C, 2 C) the recurrent branch; `in_bias [2 C]` is added to their sums.  Per token t and channel c:
//
//   x_t   = recurrent branch                                u_t = conv_bias + sum_j taps[c][K-1-j] * x_(t-j)
//   r_t   = sigmoid(Ra[b] u_t[block b] + ra_bias)           i_t = sigmoid(Ri[b] u_t[block b] + ri_bias)
//   a_t   = exp(-c r_t softplus(lam))                       S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t
//   out_t = S_t * gelu_tanh(gate branch)
//
// where the channels are cut into equal blocks, Ra[b], Ri[b] are square matrices of one block and c is a
// constant of the model (`sharpness`).  Everything
// is float32; `out` is rounded once to the compute dtype for the output projection.  A request's state is
// `[K][C]` floats: row 0 is S, rows 1 .. K-1 the last K-1 inputs x of the convolution, oldest first.  An entry
// that starts its sequence starts from zeros.
//
// Three kernels.  `conv`: a thread per (token, channel), one token per grid column, forms u (the convolution reaches back into the entry's
// earlier tokens of this step or into the state) and leaves it in scratch.  `gates`: a CTA takes 16 tokens of one
// block, holds their u in shared memory and forms 64 channels' two gates, reading each weight once for the 16
// tokens; it leaves a_t and the driven term in scratch.  `scan`: a CTA per
// (entry, 32 channels) walks the entry's tokens in order, then leaves S and the convolution's history in the
// slot.  A token's arithmetic is the same whatever the step holds, so float32 results do not depend on the cut.
#include "common.cuh"

#include <algorithm>

constexpr int GATE_TOKENS = 16;
constexpr int GATE_THREADS = 64;
constexpr int SCAN_WARPS = 16;  // warps of a scan CTA: all fetch, one walks
constexpr int SCAN_TILE = 128;  // tokens that a scan CTA holds in shared memory at a time
constexpr int SCAN_SMEM = 3 * SCAN_TILE * 32 * static_cast<int>(sizeof(float));
constexpr int MAX_TAPS = 16;

struct RecurrentArgs {
    const float* proj;  // [splits][tokens][2 * channels]
    int splits;
    size_t split_stride;
    const float* in_bias;    // [2 * channels]
    const float* taps;       // [channels][K]
    const float* conv_bias;  // [channels]
    const float* ra_t;       // [blocks][block_width (in)][block_width (out)]
    const float* ra_bias;    // [channels]
    const float* ri_t;
    const float* ri_bias;
    const float* lam;  // [channels]
    const int* entry_of_token;
    const int* cu_tokens;
    const int* state_slots;
    const int* fresh;
    float* state;   // [slots + 1][K][channels]
    float* decay;   // scratch [tokens][channels]: a_t
    float* driven;  // scratch [tokens][channels]: sqrt(1 - a_t^2) i_t u_t
    float* conv;    // scratch [tokens][channels]: u_t
    void* out;      // [tokens][channels]
    int tokens, entries, channels, blocks, taps_count;
    float sharpness;  // c of a_t = exp(-c r_t softplus(lam))
};

// The recurrent branch's input of token `t` at channel c (projection sum + bias).
__device__ __forceinline__ float branch_input(const RecurrentArgs& a, int t, int column) {
    const float* src = a.proj + static_cast<size_t>(t) * 2 * a.channels + column;
    float v = 0.0f;
    for (int s = 0; s < a.splits; ++s) v += src[s * a.split_stride];
    return v + a.in_bias[column];
}

__global__ void __launch_bounds__(256) rglru_conv_kernel(RecurrentArgs a) {
    const int K = a.taps_count;
    const int t = blockIdx.x;
    const int c = blockIdx.y * 256 + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (c >= a.channels) return;
    const int entry = a.entry_of_token[t];
    const int n = t - a.cu_tokens[entry];  // tokens of this entry in front of t
    const float* history = a.fresh[entry] ? nullptr : a.state + (static_cast<size_t>(a.state_slots[entry]) * K + 1) * a.channels;
    float u = a.conv_bias[c];
    for (int back = 0; back < K; ++back) {
        float x = 0.0f;
        if (n - back >= 0) x = branch_input(a, t - back, a.channels + c);
        else if (history) x = history[static_cast<size_t>(n - back + K - 1) * a.channels + c];
        u = fmaf(a.taps[static_cast<size_t>(c) * K + (K - 1 - back)], x, u);
    }
    a.conv[static_cast<size_t>(t) * a.channels + c] = u;
}

__global__ void __launch_bounds__(GATE_THREADS) rglru_gates_kernel(RecurrentArgs a) {
    extern __shared__ __align__(16) float u_tile[];  // [block_width][GATE_TOKENS]: a channel's 16 tokens side by side
    const int width = a.channels / a.blocks;
    const int chunks = (width + GATE_THREADS - 1) / GATE_THREADS;
    const int block = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
    const int first_token = blockIdx.x * GATE_TOKENS;
    pdl_trigger();
    pdl_wait();
#pragma unroll 4
    for (int idx = threadIdx.x; idx < GATE_TOKENS * width; idx += GATE_THREADS) {
        const int tok = idx / width, j = idx % width;
        const int t = first_token + tok;
        u_tile[j * GATE_TOKENS + tok] = t < a.tokens ? a.conv[static_cast<size_t>(t) * a.channels + block * width + j] : 0.0f;
    }
    __syncthreads();
    const int k = chunk * GATE_THREADS + threadIdx.x;
    if (k >= width) return;
    const int c = block * width + k;
    float r[GATE_TOKENS], g[GATE_TOKENS];
#pragma unroll
    for (int tok = 0; tok < GATE_TOKENS; ++tok) r[tok] = a.ra_bias[c], g[tok] = a.ri_bias[c];
    const float* wr = a.ra_t + static_cast<size_t>(block) * width * width + k;
    const float* wi = a.ri_t + static_cast<size_t>(block) * width * width + k;
#pragma unroll 8
    for (int j = 0; j < width; ++j) {
        const float r_weight = wr[static_cast<size_t>(j) * width], i_weight = wi[static_cast<size_t>(j) * width];
        const float4* u4 = reinterpret_cast<const float4*>(u_tile + j * GATE_TOKENS);
#pragma unroll
        for (int q = 0; q < GATE_TOKENS / 4; ++q) {
            const float4 u = u4[q];  // the same address for all lanes: one broadcast read of four tokens
            r[4 * q] = fmaf(r_weight, u.x, r[4 * q]), g[4 * q] = fmaf(i_weight, u.x, g[4 * q]);
            r[4 * q + 1] = fmaf(r_weight, u.y, r[4 * q + 1]), g[4 * q + 1] = fmaf(i_weight, u.y, g[4 * q + 1]);
            r[4 * q + 2] = fmaf(r_weight, u.z, r[4 * q + 2]), g[4 * q + 2] = fmaf(i_weight, u.z, g[4 * q + 2]);
            r[4 * q + 3] = fmaf(r_weight, u.w, r[4 * q + 3]), g[4 * q + 3] = fmaf(i_weight, u.w, g[4 * q + 3]);
        }
    }
    const float lam = a.lam[c];
    const float rate = -a.sharpness * (lam > 20.0f ? lam : log1pf(expf(lam)));  // -c softplus(lam)
#pragma unroll
    for (int tok = 0; tok < GATE_TOKENS; ++tok) {
        const int t = first_token + tok;
        if (t >= a.tokens) break;
        const float recur = 1.0f / (1.0f + expf(-r[tok])), input = 1.0f / (1.0f + expf(-g[tok]));
        const float log_a = rate * recur;
        const size_t at = static_cast<size_t>(t) * a.channels + c;
        // 1 + expm1(x) and not exp(x): near x = 0 the sum is the float nearest to the true decay, where expf may be off by
        // two ulp in one direction, which a state that lives for a thousand tokens multiplies up token by token
        a.decay[at] = 1.0f + expm1f(log_a);
        a.driven[at] = sqrtf(-expm1f(2.0f * log_a)) * input * u_tile[k * GATE_TOKENS + tok];  // sqrt(1 - a^2) i u
    }
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A CTA owns 32 channels of one entry.  Its sixteen warps fetch a tile of 128 tokens (decay, driven term, gate
// branch) while the tile before is being worked on, and apply the gate's activation; warp 0 alone then walks the
// tile in order, one channel per lane, which is all that is serial: one multiply-add per token.
template <typename OutT>
__global__ void __launch_bounds__(SCAN_WARPS * 32) rglru_scan_kernel(RecurrentArgs a) {
    extern __shared__ float scan_tiles[];
    float (*s_decay)[32] = reinterpret_cast<float (*)[32]>(scan_tiles);
    float (*s_state)[32] = s_decay + SCAN_TILE;
    float (*s_gate)[32] = s_state + SCAN_TILE;
    constexpr int PER_THREAD = SCAN_TILE / SCAN_WARPS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 32 + lane;
    const bool live = c < a.channels;
    const int entry = blockIdx.y;
    const int K = a.taps_count;
    pdl_trigger();
    pdl_wait();
    const int begin = a.cu_tokens[entry], end = a.cu_tokens[entry + 1];
    const int count = end - begin;
    float* slot = a.state + static_cast<size_t>(a.state_slots[entry]) * K * a.channels;
    const bool fresh = a.fresh[entry] != 0;
    float state = 0.0f;
    float history[MAX_TAPS - 1];
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i) history[i] = 0.0f;
    if (warp == 0 && live && !fresh) {
        state = slot[c];
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < K - 1) history[i] = slot[static_cast<size_t>(1 + i) * a.channels + c];
    }
    OutT* out = static_cast<OutT*>(a.out);
    const float gate_bias = live ? a.in_bias[c] : 0.0f;
    float r_decay[PER_THREAD], r_driven[PER_THREAD], r_gate[PER_THREAD];
    // All loads of a tile are issued before any is used: the partial sums are walked split by split, not token by token.
    auto fetch = [&](int tile_begin) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int t = tile_begin + warp + i * SCAN_WARPS;
            const bool there = t < end && live;
            const size_t at = static_cast<size_t>(there ? t : begin) * a.channels + (live ? c : 0);
            r_decay[i] = there ? a.decay[at] : 0.0f;
            r_driven[i] = there ? a.driven[at] : 0.0f;
            r_gate[i] = 0.0f;
        }
        for (int s = 0; s < a.splits; ++s) {
#pragma unroll
            for (int i = 0; i < PER_THREAD; ++i) {
                const int t = tile_begin + warp + i * SCAN_WARPS;
                if (t < end && live) r_gate[i] += a.proj[s * a.split_stride + static_cast<size_t>(t) * 2 * a.channels + c];
            }
        }
    };
    fetch(begin);
    for (int tile_begin = begin; tile_begin < end; tile_begin += SCAN_TILE) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int tok = warp + i * SCAN_WARPS;
            s_decay[tok][lane] = r_decay[i];
            s_state[tok][lane] = r_driven[i];
            s_gate[tok][lane] = gelu_tanh(r_gate[i] + gate_bias);
        }
        __syncthreads();
        fetch(tile_begin + SCAN_TILE);  // the next tile's loads are in flight under the serial walk
        const int n = min(SCAN_TILE, end - tile_begin);
        if (warp == 0) {
            // eight tokens at a time: their decays and driven terms are read first, then the chain of multiply-adds runs
            for (int tok0 = 0; tok0 < n; tok0 += 8) {
                float decay8[8], driven8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) decay8[i] = s_decay[tok0 + i][lane], driven8[i] = s_state[tok0 + i][lane];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (tok0 + i < n) state = fmaf(decay8[i], state, driven8[i]);
                    driven8[i] = state;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) s_state[tok0 + i][lane] = driven8[i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int tok = warp + i * SCAN_WARPS;
            if (tok < n && live)
                out[static_cast<size_t>(tile_begin + tok) * a.channels + c] = from_float<OutT>(s_state[tok][lane] * s_gate[tok][lane]);
        }
        __syncthreads();
    }
    if (warp != 0 || !live) return;
    slot[c] = state;
    // The convolution's history after this entry: the inputs of the sequence's last K - 1 positions, of which
    // the entry brought the last `count` (or all of them).
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i) {
        if (i >= K - 1) break;
        const int n = count - (K - 1) + i;  // index among the entry's tokens, negative: older than the entry
        float x;
        if (n >= 0) {
            x = branch_input(a, begin + n, a.channels + c);
        } else {
            x = 0.0f;  // history[i + count], picked without a dynamic register index
#pragma unroll
            for (int h = 0; h < MAX_TAPS - 1; ++h)
                if (h == i + count) x = history[h];
        }
        slot[static_cast<size_t>(1 + i) * a.channels + c] = x;
    }
}

static SharedMemoryOptIn g_gates_opt_in;

ME_EXPORT int me_rglru(const float* proj, int splits, long long split_stride, const float* in_bias, const float* taps,
                       const float* conv_bias, const float* ra_t, const float* ra_bias, const float* ri_t,
                       const float* ri_bias, const float* lam, const int* entry_of_token, const int* cu_tokens,
                       const int* state_slots, const int* fresh, float* state, float* decay, float* driven, float* conv,
                       void* out,
                       int out_type, int tokens, int entries, int channels, int blocks, int taps_count,
                       float sharpness, cudaStream_t stream) {
    if (tokens <= 0 || entries <= 0) return 0;
    if (blocks < 1 || channels % blocks || taps_count < 1) return ME_ERR_ARGUMENT;
    if (taps_count > MAX_TAPS) return ME_ERR_UNSUPPORTED;
    const int width = channels / blocks;
    const size_t smem = static_cast<size_t>(GATE_TOKENS) * width * sizeof(float);
    if (smem > 200 * 1024) return ME_ERR_UNSUPPORTED;
    RecurrentArgs a{proj, splits, (size_t)split_stride, in_bias, taps, conv_bias, ra_t, ra_bias, ri_t, ri_bias, lam,
                    entry_of_token, cu_tokens, state_slots, fresh, state, decay, driven, conv, out, tokens, entries, channels,
                    blocks, taps_count, sharpness};
    if (smem > 48 * 1024) {
        const int status = g_gates_opt_in(rglru_gates_kernel, static_cast<int>(smem));
        if (status) return status;
    }
    const int chunks = (width + GATE_THREADS - 1) / GATE_THREADS;
    const dim3 gate_grid((tokens + GATE_TOKENS - 1) / GATE_TOKENS, blocks * chunks);
    const dim3 conv_grid(tokens, (channels + 255) / 256);
    int status = launch_kernel(rglru_conv_kernel, conv_grid, 256, 0, stream, a);
    if (status) return status;
    status = launch_kernel(rglru_gates_kernel, gate_grid, GATE_THREADS, smem, stream, a);
    if (status) return status;
    const dim3 scan_grid((channels + 31) / 32, entries);
    if (out_type == ME_BF16) {
        static SharedMemoryOptIn opt_in;
        if (const int e = opt_in(rglru_scan_kernel<__nv_bfloat16>, SCAN_SMEM)) return e;
        return launch_kernel(rglru_scan_kernel<__nv_bfloat16>, scan_grid, SCAN_WARPS * 32, SCAN_SMEM, stream, a);
    }
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(rglru_scan_kernel<float>, SCAN_SMEM)) return e;
    return launch_kernel(rglru_scan_kernel<float>, scan_grid, SCAN_WARPS * 32, SCAN_SMEM, stream, a);
}

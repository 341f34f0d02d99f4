// The router of a feed-forward made of many small units ("experts") of which a token uses a few.
//
// Per token: z = W_r h in float32 (h in the compute dtype, W_r float32), s = sigmoid(z).  The units form
// `group_count` equal groups of neighbours; a group's value is the sum of its two largest scores (of its
// only score when a group is a single unit) and only units of the `group_keep` best groups are eligible.
// Among those the `top` largest scores are chosen; their weights are s / (sum of the chosen s + 1e-20) *
// weight_scale.  Ties go to the lower index.  The kernel leaves a dense map `weights [T][units]` (zero for
// units that were not chosen), and the chosen units and their weights as lists `[T][top]`.
//
// One block per token: warp w forms the scores of units w, w + 4, ...; one thread then chooses.  The sums
// run over the columns in a fixed order, so a token's choice never depends on the rest of the batch.
#include "common.cuh"

constexpr int ROUTE_WARPS = 4;
constexpr int MAX_UNITS = 1024;

struct RouteArgs {
    const void* h;        // [tokens][hidden]
    const float* router;  // [units][hidden]
    float* weights;       // [tokens][units]
    int* chosen;          // [tokens][top]
    float* chosen_weight; // [tokens][top]
    int tokens, hidden, units, top, group_count, group_keep;
    float weight_scale;
};

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_kernel(RouteArgs a) {
    __shared__ float score[MAX_UNITS];
    __shared__ unsigned char eligible[MAX_UNITS];
    const int token = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    const T* h = static_cast<const T*>(a.h) + static_cast<size_t>(token) * a.hidden;
    for (int unit = warp; unit < a.units; unit += ROUTE_WARPS) {
        const float* w = a.router + static_cast<size_t>(unit) * a.hidden;
        float sum = 0.0f;
        for (int i = lane; i < a.hidden; i += 32) sum = fmaf(to_float(h[i]), w[i], sum);
        sum = warp_sum(sum);
        if (lane == 0) score[unit] = 1.0f / (1.0f + expf(-sum));
    }
    for (int unit = threadIdx.x; unit < a.units; unit += ROUTE_WARPS * 32) {
        eligible[unit] = 0;
        a.weights[static_cast<size_t>(token) * a.units + unit] = 0.0f;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    const int per = a.units / a.group_count;
    // The best groups, one at a time (group counts are small).
    for (int round = 0; round < a.group_keep; ++round) {
        int best = -1;
        float best_value = -INFINITY;
        for (int g = 0; g < a.group_count; ++g) {
            if (eligible[g * per]) continue;  // taken in an earlier round
            float first = -INFINITY, second = -INFINITY;
            for (int u = g * per; u < (g + 1) * per; ++u) {
                const float s = score[u];
                if (s > first) second = first, first = s;
                else if (s > second) second = s;
            }
            const float value = per > 1 ? first + second : first;
            if (value > best_value) best_value = value, best = g;
        }
        if (best < 0) break;
        for (int u = best * per; u < (best + 1) * per; ++u) eligible[u] = 1;
    }
    float total = 0.0f;
    int* chosen = a.chosen + static_cast<size_t>(token) * a.top;
    float* chosen_weight = a.chosen_weight + static_cast<size_t>(token) * a.top;
    for (int round = 0; round < a.top; ++round) {
        int best = -1;
        float best_score = -INFINITY;
        for (int u = 0; u < a.units; ++u)
            if (eligible[u] == 1 && score[u] > best_score) best_score = score[u], best = u;
        chosen[round] = best;
        if (best < 0) continue;
        eligible[best] = 2;
        total += best_score;
    }
    const float inv = a.weight_scale / (total + 1e-20f);
    for (int round = 0; round < a.top; ++round) {
        const int u = chosen[round];
        const float weight = u >= 0 ? score[u] * inv : 0.0f;
        chosen_weight[round] = weight;
        if (u >= 0) a.weights[static_cast<size_t>(token) * a.units + u] = weight;
    }
}

ME_EXPORT int me_route(const void* h, int h_type, const float* router, float* weights, int* chosen,
                       float* chosen_weight, int tokens, int hidden, int units, int top, int group_count,
                       int group_keep, float weight_scale, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (units < 1 || units > MAX_UNITS) return ME_ERR_UNSUPPORTED;
    if (group_count < 1 || units % group_count || group_keep < 1 || group_keep > group_count || top < 1 ||
        top > group_keep * (units / group_count))
        return ME_ERR_ARGUMENT;
    RouteArgs a{h, router, weights, chosen, chosen_weight, tokens, hidden, units, top, group_count, group_keep, weight_scale};
    if (h_type == ME_BF16) return launch_kernel(route_kernel<__nv_bfloat16>, tokens, ROUTE_WARPS * 32, 0, stream, a);
    return launch_kernel(route_kernel<float>, tokens, ROUTE_WARPS * 32, 0, stream, a);
}

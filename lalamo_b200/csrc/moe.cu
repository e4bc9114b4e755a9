// Routed feed-forward: a router that scores experts (sigmoid or softmax), restricts the choice to the best
// groups of neighbouring experts, and picks the `top` largest; gated experts evaluated per (token, chosen
// expert) with the expert's weights streamed once per pair; and the weighted sum of the experts' outputs.
// Router, scores and the weighted sum are 32-bit.
#include "common.cuh"

namespace lb {

// The lane-wise best (largest value, lowest index among equals) over a warp; every lane gets it.
__device__ __forceinline__ void warp_argmax(float& value, int& index) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other_value > value || (other_value == value && other_index < index)) {
            value = other_value;
            index = other_index;
        }
    }
}

// One warp per token.
//   z[e] = x . router[e]  (32-bit);   s[e] = sigmoid(z[e])   (score_kind 0)  or softmax(z)[e]   (score_kind 1)
//   experts form `group_count` equal groups of neighbours; a group's score is the sum of its two largest s (of its
//   only one, in groups of one); experts outside the best `group_keep` groups cannot be chosen;
//   chosen[t, :] = the `top` eligible experts of largest s, in that order; weights[t, :] = their s (divided by their
//   sum if `renormalize`), times `weight_scale`.
// Shared memory per warp: s[experts], candidates[experts], group score[group_count].
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router, int* __restrict__ chosen, float* __restrict__ weights,
                                 int tokens, int width, int experts, int top, int group_count, int group_keep, int score_kind, int renormalize,
                                 float weight_scale) {
    extern __shared__ float shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int token = blockIdx.x * warps + warp;
    if (token >= tokens) return;
    float* scores = shared + static_cast<size_t>(warp) * (2 * experts + group_count);
    float* candidates = scores + experts;
    float* group_score = candidates + experts;
    const T* row = x + static_cast<size_t>(token) * width;
    for (int e = 0; e < experts; ++e) {
        const float* w = router + static_cast<size_t>(e) * width;
        float dot = 0.0f;
        for (int d = lane; d < width; d += 32) dot += to_float(row[d]) * w[d];
        dot = warp_sum(dot);
        if (lane == 0) scores[e] = dot;
    }
    __syncwarp();
    if (score_kind == 1) {
        float largest = -INFINITY;
        for (int e = lane; e < experts; e += 32) largest = fmaxf(largest, scores[e]);
        largest = warp_max(largest);
        float total = 0.0f;
        for (int e = lane; e < experts; e += 32) total += expf(scores[e] - largest);
        total = warp_sum(total);
        for (int e = lane; e < experts; e += 32) scores[e] = expf(scores[e] - largest) / total;
    } else {
        for (int e = lane; e < experts; e += 32) scores[e] = 1.0f / (1.0f + expf(-scores[e]));
    }
    __syncwarp();
    const int members = experts / group_count;
    for (int group = lane; group < group_count; group += 32) {
        float first = -INFINITY, second = -INFINITY;
        for (int m = 0; m < members; ++m) {
            const float s = scores[group * members + m];
            if (s > first) {
                second = first;
                first = s;
            } else if (s > second) {
                second = s;
            }
        }
        group_score[group] = members >= 2 ? first + second : first;
    }
    for (int e = lane; e < experts; e += 32) candidates[e] = -INFINITY;
    __syncwarp();
    for (int round = 0; round < group_keep; ++round) {
        float best = -INFINITY;
        int best_group = 0x7fffffff;
        for (int group = lane; group < group_count; group += 32) {
            const float s = group_score[group];
            if (s > best) {   // ascending scan: the lowest index among equals stays
                best = s;
                best_group = group;
            }
        }
        warp_argmax(best, best_group);
        if (best_group == 0x7fffffff) break;
        for (int m = lane; m < members; m += 32) candidates[best_group * members + m] = scores[best_group * members + m];
        if (lane == 0) group_score[best_group] = -INFINITY;
        __syncwarp();
    }
    float total = 0.0f;
    for (int round = 0; round < top; ++round) {
        float best = -INFINITY;
        int best_expert = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float s = candidates[e];
            if (s > best) {
                best = s;
                best_expert = e;
            }
        }
        warp_argmax(best, best_expert);
        if (best_expert == 0x7fffffff) best_expert = 0, best = 0.0f;   // fewer eligible experts than `top`: a weight of zero
        total += best;
        if (lane == 0) {
            chosen[static_cast<size_t>(token) * top + round] = best_expert;
            weights[static_cast<size_t>(token) * top + round] = best;
            if (best_expert < experts) candidates[best_expert] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float factor = (renormalize && total > 0.0f ? 1.0f / total : 1.0f) * weight_scale;
        if (factor != 1.0f)
            for (int round = 0; round < top; ++round) weights[static_cast<size_t>(token) * top + round] *= factor;
    }
}

__device__ __forceinline__ float moe_activate(float v, int activation) {
    if (activation == 0) return v / (1.0f + expf(-v));                                   // silu
    if (activation == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));    // gelu (exact)
    return v;
}

// One block per (token, chosen expert) pair p: hidden = act(W_gate[e] x) * (W_up[e] x), rounded to T; out[p] = W_down[e] hidden
// in 32-bit.  A warp per output row, lanes along the row, sums in lane order then over the warp.
//   gate, up [experts, ff, width];  down [experts, width, ff];  out [pairs, width] (32-bit)
template <typename T>
__global__ void moe_expert_stream_kernel(const T* __restrict__ x, const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ down,
                                         const int* __restrict__ chosen, float* __restrict__ out, int top, int width, int ff, int experts,
                                         int activation) {
    extern __shared__ float shared[];
    float* x_s = shared;           // width
    float* hidden = shared + width;   // ff
    const int pair = blockIdx.x;
    const int token = pair / top;
    const int expert = chosen[pair];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* dst = out + static_cast<size_t>(pair) * width;
    if (expert < 0 || expert >= experts) {
        for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = 0.0f;
        return;
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) x_s[d] = to_float(x[static_cast<size_t>(token) * width + d]);
    __syncthreads();
    const T* gate_rows = gate + static_cast<size_t>(expert) * ff * width;
    const T* up_rows = up + static_cast<size_t>(expert) * ff * width;
    for (int f = warp; f < ff; f += warps) {
        const T* g_row = gate_rows + static_cast<size_t>(f) * width;
        const T* u_row = up_rows + static_cast<size_t>(f) * width;
        float g = 0.0f, u = 0.0f;
        for (int d = lane; d < width; d += 32) {
            g += x_s[d] * to_float(g_row[d]);
            u += x_s[d] * to_float(u_row[d]);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) hidden[f] = round_to<T>(round_to<T>(moe_activate(round_to<T>(g), activation)) * round_to<T>(u));
    }
    __syncthreads();
    const T* down_rows = down + static_cast<size_t>(expert) * width * ff;
    for (int r = warp; r < width; r += warps) {
        const T* d_row = down_rows + static_cast<size_t>(r) * ff;
        float sum = 0.0f;
        for (int f = lane; f < ff; f += 32) sum += hidden[f] * to_float(d_row[f]);
        sum = warp_sum(sum);
        if (lane == 0) dst[r] = sum;
    }
}

// out[t, :] = T(sum_k weights[t, k] * expert_out[t * top + k, :]), added in the order of k.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ expert_out, const float* __restrict__ weights, T* __restrict__ out, int top, int width) {
    const int token = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) sum += weights[static_cast<size_t>(token) * top + k] * expert_out[(static_cast<size_t>(token) * top + k) * width + d];
        out[static_cast<size_t>(token) * width + d] = from_float<T>(sum);
    }
}

}  // namespace lb

extern "C" {

int lb_moe_route(const void* x, const float* router, int* chosen, float* weights, int tokens, int width, int experts, int top, int group_count,
                 int group_keep, int score_kind, int renormalize, float weight_scale, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (experts < 1 || top < 1 || top > experts || group_count < 1 || experts % group_count != 0 || group_keep < 1 || group_keep > group_count) return -2;
    constexpr int kWarps = 4;
    const size_t shared = static_cast<size_t>(kWarps) * (2 * experts + group_count) * sizeof(float);
    if (shared > 48 * 1024) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        lb::moe_route_kernel<T><<<(tokens + kWarps - 1) / kWarps, 32 * kWarps, shared, stream>>>(
            static_cast<const T*>(x), router, chosen, weights, tokens, width, experts, top, group_count, group_keep, score_kind, renormalize, weight_scale);
    })
    return LB_LAUNCH_RESULT();
}

int lb_moe_expert_stream(const void* x, const void* gate, const void* up, const void* down, const int* chosen, float* out, int pairs, int top,
                         int width, int ff, int experts, int activation, int dtype, cudaStream_t stream) {
    if (pairs == 0) return 0;
    const size_t shared = (static_cast<size_t>(width) + ff) * sizeof(float);
    if (shared > 200 * 1024) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        auto kernel = lb::moe_expert_stream_kernel<T>;
        if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        kernel<<<pairs, 256, shared, stream>>>(static_cast<const T*>(x), static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<const T*>(down),
                                               chosen, out, top, width, ff, experts, activation);
    })
    return LB_LAUNCH_RESULT();
}

int lb_moe_combine(const float* expert_out, const float* weights, void* out, int tokens, int top, int width, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LB_DISPATCH_DTYPE(dtype, {
        lb::moe_combine_kernel<T><<<tokens, 256, 0, stream>>>(expert_out, weights, static_cast<T*>(out), top, width);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"

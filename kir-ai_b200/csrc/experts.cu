// Routing for a feed-forward made of small experts, of which every token uses a few.
//
//   router_gates   logits z = W_router x in 32-bit; the `top` largest are chosen (the lower index wins a tie) and the
//                  token's weights are the softmax over the chosen logits alone.  The result is the dense matrix
//                  gates [T, experts], zero where an expert was not chosen, plus the chosen ids and weights.
//   relu2_gate     hidden[t, e * ff + j] = relu(up[t, e * ff + j])^2 * gates[t, e]: with the experts' up matrices
//                  stacked along the rows and their down matrices side by side along the columns, the product
//                  hidden W_down^T is the weighted sum of the chosen experts' outputs, and an expert that was not
//                  chosen contributes exact zeros.
//
// Nothing here waits for the host or depends on how many tokens an expert drew, so a step can be captured in a graph.
#include "common.cuh"

#define ROUTER_WARPS 4

template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_gates_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ router, float* __restrict__ gates,
                    int* __restrict__ chosen_ids, float* __restrict__ chosen_weights, int hidden, int experts, int top) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float logits_s[];  // [experts]
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* row = x + (size_t)token * x_stride;
    for (int e = warp; e < experts; e += ROUTER_WARPS) {
        const float* w = router + (size_t)e * hidden;
        float dot = 0.0f;
        for (int i = lane; i < hidden; i += 32) dot = fmaf(to_f32<T>(row[i]), w[i], dot);
        dot = warp_sum(dot);
        if (lane == 0) logits_s[e] = dot;
    }
    __syncthreads();
    float* out = gates + (size_t)token * experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) out[e] = 0.0f;
    __syncthreads();
    if (warp != 0) return;
    // warp 0 picks the `top` largest one after the other; a chosen logit is replaced by -inf in shared memory after its
    // value went into the lane-0 registers below
    float best_first = 0.0f, denom = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float z = logits_s[e];
            if (z > best || (z == best && e < best_e)) {
                best = z;
                best_e = e;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
            if (other > best || (other == best && other_e < best_e)) {
                best = other;
                best_e = other_e;
            }
        }
        if (best_e == 0x7fffffff) break;  // fewer finite logits than `top` (NaN rows): the rest stays zero
        if (k == 0) best_first = best;
        const float weight = expf(best - best_first);  // the first chosen logit is the largest
        denom += weight;
        if (lane == 0) {
            out[best_e] = weight;
            if (chosen_ids) chosen_ids[(size_t)token * top + k] = best_e;
            if (chosen_weights) chosen_weights[(size_t)token * top + k] = weight;
            logits_s[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    __syncwarp();
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    for (int e = lane; e < experts; e += 32) out[e] *= inv;
    if (chosen_weights)
        for (int k = lane; k < top; k += 32) chosen_weights[(size_t)token * top + k] *= inv;
}

template <typename T>
static int router_gates_launch(const void* x, long x_stride, const float* router, float* gates, int* chosen_ids,
                               float* chosen_weights, int tokens, int hidden, int experts, int top, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts || hidden <= 0 || experts > 8192) return KIRAI_ERR_BAD_SIZE;
    return launch_pdl(router_gates_kernel<T>, dim3(tokens), dim3(ROUTER_WARPS * 32), (size_t)experts * sizeof(float), stream, 1u,
                      (const T*)x, x_stride, router, gates, chosen_ids, chosen_weights, hidden, experts, top);
}

KIRAI_EXPORT int kirai_router_gates_f32(const void* x, long x_stride, const float* router, float* gates, int* chosen_ids,
                                        float* chosen_weights, int tokens, int hidden, int experts, int top, cudaStream_t stream) {
    return router_gates_launch<float>(x, x_stride, router, gates, chosen_ids, chosen_weights, tokens, hidden, experts, top, stream);
}
KIRAI_EXPORT int kirai_router_gates_bf16(const void* x, long x_stride, const float* router, float* gates, int* chosen_ids,
                                         float* chosen_weights, int tokens, int hidden, int experts, int top, cudaStream_t stream) {
    return router_gates_launch<bf16>(x, x_stride, router, gates, chosen_ids, chosen_weights, tokens, hidden, experts, top, stream);
}

// activation: 0 = relu(z)^2
template <typename T>
__global__ void expert_activation_gate_kernel(T* __restrict__ up, const float* __restrict__ gates, long rows, int experts, int ff) {
    pdl_launch_dependents();
    pdl_wait();
    const long width = (long)experts * ff;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * width) return;
    const long row = idx / width;
    const int expert = (int)((idx - row * width) / ff);
    const float gate = gates[row * experts + expert];
    float z = to_f32<T>(up[idx]);
    z = z > 0.0f ? z * z : 0.0f;
    up[idx] = from_f32<T>(gate == 0.0f ? 0.0f : z * gate);  // an expert that was not chosen gives zeros whatever it computed
}

template <typename T>
static int expert_activation_gate_launch(void* up, const float* gates, int rows, int experts, int ff, cudaStream_t stream) {
    const long total = (long)rows * experts * ff;
    if (total <= 0) return 0;
    return launch_pdl(expert_activation_gate_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1u, (T*)up,
                      gates, (long)rows, experts, ff);
}

// up [T, experts * ff] in place: relu(z)^2 times the token's gate of the column's expert.
KIRAI_EXPORT int kirai_relu2_gate_f32(void* up, const float* gates, int rows, int experts, int ff, cudaStream_t stream) {
    return expert_activation_gate_launch<float>(up, gates, rows, experts, ff, stream);
}
KIRAI_EXPORT int kirai_relu2_gate_bf16(void* up, const float* gates, int rows, int experts, int ff, cudaStream_t stream) {
    return expert_activation_gate_launch<bf16>(up, gates, rows, experts, ff, stream);
}

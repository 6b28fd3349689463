// Routed experts (mixture of experts): the router, and the experts' activation with the routing weights.
//
// moe_route_kernel   per token: logits z = W_r x in 32-bit (x may be the compute dtype's rounding of the
//                    normed stream; W_r is held in float32), scores s = sigmoid(z).  Experts form `groups`
//                    equal groups of neighbours; a group's score is the sum of its two largest scores (of
//                    its one score when a group is one expert) and only experts of the `keep` best groups
//                    may be chosen (groups = 0: no such limit).  The `top` largest allowed scores are
//                    chosen (ties go to the lower index); their weights are s / (sum of the chosen s +
//                    1e-20) * route_scale.  Written as a dense row of float32 weights [experts] (zero for
//                    experts that were not chosen) and, optionally, as the lists ids [top], weights [top].
// moe_act_kernel     from the float32 product [T, experts * 2 * ff] of the token rows with every expert's
//                    [gate; up] matrix: act[t, e*ff + f] = w[t, e] * g * sigmoid(alpha g) * (u + 1) with
//                    g = min(gate, limit), u = clamp(up, -limit, limit), in the compute dtype, zero where
//                    w[t, e] is zero.  The experts' down matrices stand side by side along the input axis,
//                    so ONE product of `act` with them is the weighted sum of the chosen experts' outputs.
#include "common.cuh"
#include <math_constants.h>

#define MOE_ROUTE_THREADS 128

template <typename TX>
__global__ void moe_route_kernel(const TX* __restrict__ x, const float* __restrict__ wr, float* __restrict__ dense,
                                 int32_t* __restrict__ ids, float* __restrict__ weights, int W, int E, int top,
                                 int groups, int keep, float route_scale) {
    pdl_begin();
    extern __shared__ float smem[];
    float* xs = smem;                    // [W]
    float* score = xs + W;               // [E]
    float* gscore = score + E;           // [groups]
    int* allowed = reinterpret_cast<int*>(gscore + (groups > 0 ? groups : 1));      // [E]
    const long long t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < W; i += blockDim.x) xs[i] = to_f32(x[t * W + i]);
    __syncthreads();
    for (int e = warp; e < E; e += MOE_ROUTE_THREADS / 32) {
        const float* w = wr + static_cast<size_t>(e) * W;
        float dot = 0.0f;
        for (int i = lane; i < W; i += 32) dot += w[i] * xs[i];
        dot = warp_sum(dot);
        if (lane == 0) score[e] = 1.0f / (1.0f + expf(-dot));
    }
    __syncthreads();
    const int per = groups > 0 ? E / groups : E;
    if (groups > 0) {
        for (int g = tid; g < groups; g += blockDim.x) {
            float a = -1.0f, b = -1.0f;              // the two largest (scores are in (0, 1))
            for (int j = 0; j < per; ++j) {
                const float s = score[g * per + j];
                if (s > a) { b = a; a = s; }
                else if (s > b) b = s;
            }
            gscore[g] = per > 1 ? a + b : a;
        }
    }
    for (int e = tid; e < E; e += blockDim.x) {
        allowed[e] = groups > 0 ? 0 : 1;
        dense[t * E + e] = 0.0f;
    }
    __syncthreads();
    if (tid == 0) {
        for (int n = 0; n < keep && groups > 0; ++n) {      // the best groups, ties to the lower index
            int best = -1;
            float bs = -CUDART_INF_F;
            for (int g = 0; g < groups; ++g)
                if (gscore[g] > bs) { bs = gscore[g]; best = g; }
            if (best < 0) break;
            gscore[best] = -CUDART_INF_F;
            for (int j = 0; j < per; ++j) allowed[best * per + j] = 1;
        }
        float total = 0.0f;
        int chosen[64];
        for (int n = 0; n < top; ++n) {
            int best = -1;
            float bs = -CUDART_INF_F;
            for (int e = 0; e < E; ++e)
                if (allowed[e] && score[e] > bs) { bs = score[e]; best = e; }
            chosen[n] = best;
            if (best >= 0) {
                allowed[best] = 0;
                total += bs;
            }
        }
        const float inv = route_scale / (total + 1e-20f);
        for (int n = 0; n < top; ++n) {
            const int e = chosen[n];
            const float w = e >= 0 ? score[e] * inv : 0.0f;
            if (e >= 0) dense[t * E + e] = w;
            if (ids) {
                ids[t * top + n] = e;
                weights[t * top + n] = w;
            }
        }
    }
}

extern "C" int llm_moe_route(const void* x, int x_dtype, const float* wr, float* dense, int32_t* ids, float* weights,
                             int num_tokens, int W, int E, int top, int groups, int keep, float route_scale,
                             uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (W <= 0 || E <= 0 || top <= 0 || top > E || top > 64 || groups < 0) return LLM_REFUSED_SIZE;
    if (groups > 0 && (E % groups || keep <= 0 || keep > groups || keep * (E / groups) < top)) return LLM_REFUSED_SIZE;
    const size_t smem = (static_cast<size_t>(W) + 2 * E + (groups > 0 ? groups : 1)) * sizeof(float);
    if (smem > 48 * 1024) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (x_dtype == LLM_DT_F32)
        launch_pdl((moe_route_kernel<float>), dim3(num_tokens), dim3(MOE_ROUTE_THREADS), smem, s,
                   static_cast<const float*>(x), wr, dense, ids, weights, W, E, top, groups, keep, route_scale);
    else if (x_dtype == LLM_DT_BF16)
        launch_pdl((moe_route_kernel<bf16>), dim3(num_tokens), dim3(MOE_ROUTE_THREADS), smem, s,
                   static_cast<const bf16*>(x), wr, dense, ids, weights, W, E, top, groups, keep, route_scale);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

template <typename TO>
__global__ void moe_act_kernel(const float* __restrict__ gu, int parts, long long part_stride,
                               const float* __restrict__ dense, TO* __restrict__ act, int E, int ff, float limit,
                               float alpha, long long total) {
    pdl_begin();
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long row = idx / (static_cast<long long>(E) * ff);
    const int rest = static_cast<int>(idx - row * E * ff);
    const int e = rest / ff, f = rest - e * ff;
    const float w = dense[row * E + e];
    float out = 0.0f;
    if (w != 0.0f) {
        const float* p = gu + (row * E + e) * 2 * ff;
        float g = 0.0f, u = 0.0f;
        for (int k = 0; k < parts; ++k) {                   // the product may come as its k-splits
            g += p[k * part_stride + f];
            u += p[k * part_stride + ff + f];
        }
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        out = w * (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
    }
    act[idx] = from_f32<TO>(out);
}

extern "C" int llm_moe_act(const float* gu, int parts, long long part_stride, const float* dense, void* act,
                           int act_dtype, int num_tokens, int E, int ff, float limit, float alpha, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (E <= 0 || ff <= 0 || !(limit > 0.0f)) return LLM_REFUSED_SIZE;
    const long long total = static_cast<long long>(num_tokens) * E * ff;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return LLM_REFUSED_SIZE;
    if (parts < 1) parts = 1;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (act_dtype == LLM_DT_F32)
        launch_pdl((moe_act_kernel<float>), dim3(static_cast<unsigned>(blocks)), dim3(256), 0, s, gu, parts, part_stride,
                   dense, static_cast<float*>(act), E, ff, limit, alpha, total);
    else if (act_dtype == LLM_DT_BF16)
        launch_pdl((moe_act_kernel<bf16>), dim3(static_cast<unsigned>(blocks)), dim3(256), 0, s, gu, parts, part_stride,
                   dense, static_cast<bf16*>(act), E, ff, limit, alpha, total);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

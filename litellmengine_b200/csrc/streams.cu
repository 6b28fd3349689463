// The residual update of a pre-norm layer and the norm in front of the next sublayer, in one kernel, for
// models that keep S >= 1 copies of the residual stream ("hyper-connections"; S = 1 with unit
// coefficients is the ordinary residual stream):
//
//     x'_t = sum_s mix[s, t] x_s + out[t] * y          for all t at once       (when y is given)
//     u    = sum_t in[t] x'_t
//     o    = norm(u) * w                                layer norm (centred) or RMS norm
//
// Everything is 32-bit; o is written in the compute dtype.  streams: float32 [S, T, hidden].  y: the
// sublayer output that has not been added yet ([T, hidden], float32 or bfloat16, possibly the k-splits of
// a product, `y_parts` tensors `y_part_stride` elements apart, added in order as they are read).  A null
// `mix` is the identity, a null `outw` or `inw` all ones (in = ones: the sum of the streams, which is what
// the model's final norm reads).  `rows` picks the rows that are read (the final norm runs only where
// logits are wanted); the new streams are written back only without `rows`.  A null `w`: the streams are
// updated and nothing is normalised.  `read_stride` is the distance between the streams as they are READ: 0 at a
// model's first layer, where all streams equal the embedding that sits in stream 0 (they are then written out
// to their own places, so no kernel has to copy the embedding S times).
//
// Layer norm: mean, then the mean of the squared deviations (two passes over the row held in shared
// memory), eps inside the root.  One block per row.
#include "common.cuh"

#define ST_MAX 8

template <typename TY, typename TO>
__global__ void stream_norm_kernel(float* __restrict__ streams, long long stream_stride, long long read_stride, int S,
                                   const TY* __restrict__ y, int y_parts, long long y_part_stride,
                                   const float* __restrict__ mix, const float* __restrict__ outw,
                                   const float* __restrict__ inw, const float* __restrict__ w, float eps, int center,
                                   TO* __restrict__ out, const int32_t* __restrict__ rows, int hidden, int write_back) {
    extern __shared__ __align__(16) float smem[];
    float* u = smem;                                   // [hidden]
    float* scratch = smem + ((hidden + 7) & ~7);       // 33
    float* coef = scratch + 33;                        // mix [S*S], out [S], in [S]
    // the coefficients are weights: read before the wait for the kernel that produces y
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) coef[i] = mix ? mix[i] : ((i / S == i % S) ? 1.0f : 0.0f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        coef[S * S + i] = outw ? outw[i] : 1.0f;
        coef[S * S + S + i] = inw ? inw[i] : 1.0f;
    }
    pdl_begin();
    __syncthreads();
    const size_t src = rows ? static_cast<size_t>(rows[blockIdx.x]) : blockIdx.x;
    float* xr = streams + src * hidden;
    const TY* yr = y ? y + src * hidden : nullptr;
    float sum = 0.0f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float x[ST_MAX];
#pragma unroll
        for (int s = 0; s < ST_MAX; ++s)
            if (s < S) x[s] = xr[s * read_stride + h];
        float acc = 0.0f;
        if (yr) {
            float yv = 0.0f;
            for (int part = 0; part < y_parts; ++part) yv += to_f32(yr[part * y_part_stride + h]);
#pragma unroll
            for (int t = 0; t < ST_MAX; ++t)
                if (t < S) {
                    float nt = 0.0f;
#pragma unroll
                    for (int s = 0; s < ST_MAX; ++s)
                        if (s < S) nt += coef[s * S + t] * x[s];
                    nt += coef[S * S + t] * yv;
                    if (write_back) xr[t * stream_stride + h] = nt;
                    acc += coef[S * S + S + t] * nt;
                }
        } else {
#pragma unroll
            for (int t = 0; t < ST_MAX; ++t)
                if (t < S) {
                    acc += coef[S * S + S + t] * x[t];
                    if (write_back) xr[t * stream_stride + h] = x[t];
                }
        }
        u[h] = acc;
        sum += acc;
    }
    if (!w) return;
    float mean = 0.0f;
    if (center) mean = block_sum(sum, scratch) / static_cast<float>(hidden);
    float ss = 0.0f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float d = u[h] - mean;
        ss += d * d;
    }
    const float var = block_sum(ss, scratch) / static_cast<float>(hidden);
    const float inv = 1.0f / sqrtf(var + eps);
    TO* orow = out + static_cast<size_t>(blockIdx.x) * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) orow[h] = from_f32<TO>((u[h] - mean) * inv * w[h]);
}

extern "C" int llm_stream_norm(float* streams, long long stream_stride, long long read_stride, int S, const void* y, int y_dtype, int y_parts,
                               long long y_part_stride, const float* mix, const float* outw, const float* inw,
                               const float* w, float eps, int center, void* out, int out_dtype, const int32_t* rows,
                               int num_rows, int hidden, int write_back, uintptr_t stream) {
    if (num_rows <= 0) return LLM_OK;
    if (hidden <= 0 || S < 1 || S > ST_MAX) return LLM_REFUSED_SIZE;
    if (write_back && rows) return LLM_REFUSED_SIZE;
    if (w && !out) return LLM_REFUSED_SIZE;
    const size_t smem = (static_cast<size_t>((hidden + 7) & ~7) + 33 + S * S + 2 * S) * sizeof(float);
    if (smem > 200 * 1024) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
    if (y_parts < 1) y_parts = 1;
#define LAUNCH(TY, TO)                                                                                              \
    do {                                                                                                            \
        auto kern = stream_norm_kernel<TY, TO>;                                                                     \
        if (smem > 48 * 1024) {                                                                                     \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                                       static_cast<int>(smem));                                     \
            if (e != cudaSuccess) return static_cast<int>(e);                                                       \
        }                                                                                                           \
        launch_pdl(kern, dim3(num_rows), dim3(threads), smem, s, streams, stream_stride, read_stride, S,                         \
                   static_cast<const TY*>(y), y_parts, y_part_stride, mix, outw, inw, w, eps, center,               \
                   static_cast<TO*>(out), rows, hidden, write_back);                                                \
    } while (0)
    if (!y) y_dtype = LLM_DT_F32;
    if (!out) out_dtype = LLM_DT_F32;
    if (y_dtype == LLM_DT_F32 && out_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (y_dtype == LLM_DT_F32 && out_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (y_dtype == LLM_DT_BF16 && out_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else if (y_dtype == LLM_DT_BF16 && out_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

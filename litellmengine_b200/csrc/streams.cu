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

__device__ __forceinline__ void stream_load4(const float* p, float (&o)[4], int vec) {
    if (vec) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    } else {
        o[0] = *p; o[1] = o[2] = o[3] = 0.0f;
    }
}
__device__ __forceinline__ void stream_load4(const bf16* p, float (&o)[4], int vec) {
    if (vec) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    } else {
        o[0] = __bfloat162float(*p); o[1] = o[2] = o[3] = 0.0f;
    }
}
__device__ __forceinline__ void stream_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void stream_store4(bf16* p, float a, float b, float c, float d) {
    uint2 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(a, b);
    h[1] = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = raw;
}

// SM: the most streams this instantiation holds in registers (1, 2, 4 or 8).
template <typename TY, typename TO, int SM>
__global__ void stream_norm_kernel(float* __restrict__ streams, long long stream_stride, long long read_stride, int S,
                                   const TY* __restrict__ y, int y_parts, long long y_part_stride,
                                   const float* __restrict__ mix, const float* __restrict__ outw,
                                   const float* __restrict__ inw, const float* __restrict__ w, float eps, int center,
                                   TO* __restrict__ out, const int32_t* __restrict__ rows, int hidden, int write_back, int vec) {
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
    TO* orow = out ? out + static_cast<size_t>(blockIdx.x) * hidden : nullptr;
    float sum = 0.0f;
    // four neighbouring columns a thread and trip when the rows allow sixteen-byte accesses, else one
    const int step = vec ? 4 : 1;
    for (int h = threadIdx.x * step; h < hidden; h += blockDim.x * step) {
        float x[SM][4];
#pragma unroll
        for (int s = 0; s < SM; ++s)
            if (s < S) {
                if (vec) {
                    const float4 v = *reinterpret_cast<const float4*>(xr + s * read_stride + h);
                    x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
                } else {
                    x[s][0] = xr[s * read_stride + h];
                }
            }
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (yr) {
            float yv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int part = 0; part < y_parts; ++part) {
                float one[4];
                stream_load4(yr + part * y_part_stride + h, one, vec);
#pragma unroll
                for (int c = 0; c < 4; ++c) yv[c] += one[c];
            }
#pragma unroll
            for (int t = 0; t < SM; ++t)
                if (t < S) {
                    float nt[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int s = 0; s < SM; ++s)
                        if (s < S) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) nt[c] += coef[s * S + t] * x[s][c];
                        }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        nt[c] += coef[S * S + t] * yv[c];
                        acc[c] += coef[S * S + S + t] * nt[c];
                    }
                    if (write_back) {
                        if (vec) *reinterpret_cast<float4*>(xr + t * stream_stride + h) = make_float4(nt[0], nt[1], nt[2], nt[3]);
                        else xr[t * stream_stride + h] = nt[0];
                    }
                }
        } else {
#pragma unroll
            for (int t = 0; t < SM; ++t)
                if (t < S) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[c] += coef[S * S + S + t] * x[t][c];
                    if (write_back) {
                        if (vec) *reinterpret_cast<float4*>(xr + t * stream_stride + h) = make_float4(x[t][0], x[t][1], x[t][2], x[t][3]);
                        else xr[t * stream_stride + h] = x[t][0];
                    }
                }
        }
        if (vec) {
            *reinterpret_cast<float4*>(u + h) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            sum += (acc[0] + acc[1]) + (acc[2] + acc[3]);
        } else {
            u[h] = acc[0];
            sum += acc[0];
        }
    }
    if (!w) return;
    float mean = 0.0f;
    if (center) mean = block_sum(sum, scratch) / static_cast<float>(hidden);
    else __syncthreads();
    float ss = 0.0f;
    for (int h = threadIdx.x * step; h < hidden; h += blockDim.x * step) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (c < step) {
                const float d = u[h + c] - mean;
                ss += d * d;
            }
    }
    const float var = block_sum(ss, scratch) / static_cast<float>(hidden);
    const float inv = 1.0f / sqrtf(var + eps);
    for (int h = threadIdx.x * step; h < hidden; h += blockDim.x * step) {
        if (vec) {
            const float4 g = *reinterpret_cast<const float4*>(w + h);
            const float4 a = *reinterpret_cast<const float4*>(u + h);
            stream_store4(orow + h, (a.x - mean) * inv * g.x, (a.y - mean) * inv * g.y, (a.z - mean) * inv * g.z,
                          (a.w - mean) * inv * g.w);
        } else {
            orow[h] = from_f32<TO>((u[h] - mean) * inv * w[h]);
        }
    }
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
    // few rows (a decode step): more threads a row, up to 512 (what the widest instantiation's registers allow),
    // so that a row takes fewer trips
    int threads = hidden >= 1024 ? 256 : 128;
    if (num_rows <= 256 && hidden > 4 * threads) threads = hidden / 4 >= 512 ? 512 : ((hidden / 4 + 31) / 32) * 32;
    if (y_parts < 1) y_parts = 1;
    const int vec = hidden % 4 == 0 && aligned16(streams) && stream_stride % 4 == 0 && read_stride % 4 == 0 &&
                    (!y || (aligned16(y) && y_part_stride % 4 == 0)) && (!w || aligned16(w)) && (!out || aligned16(out));
#define LAUNCH_S(TY, TO, SMAX)                                                                                      \
    do {                                                                                                            \
        auto kern = stream_norm_kernel<TY, TO, SMAX>;                                                               \
        if (smem > 48 * 1024) {                                                                                     \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                                       static_cast<int>(smem));                                     \
            if (e != cudaSuccess) return static_cast<int>(e);                                                       \
        }                                                                                                           \
        launch_pdl(kern, dim3(num_rows), dim3(threads), smem, s, streams, stream_stride, read_stride, S,                         \
                   static_cast<const TY*>(y), y_parts, y_part_stride, mix, outw, inw, w, eps, center,               \
                   static_cast<TO*>(out), rows, hidden, write_back, vec);                                           \
    } while (0)
#define LAUNCH(TY, TO)                                                                                              \
    do {                                                                                                            \
        if (S == 1) LAUNCH_S(TY, TO, 1);                                                                            \
        else if (S == 2) LAUNCH_S(TY, TO, 2);                                                                       \
        else if (S <= 4) LAUNCH_S(TY, TO, 4);                                                                       \
        else LAUNCH_S(TY, TO, 8);                                                                                   \
    } while (0)
    if (!y) y_dtype = LLM_DT_F32;
    if (!out) out_dtype = LLM_DT_F32;
    if (y_dtype == LLM_DT_F32 && out_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (y_dtype == LLM_DT_F32 && out_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (y_dtype == LLM_DT_BF16 && out_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else if (y_dtype == LLM_DT_BF16 && out_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
#undef LAUNCH_S
    return launch_status();
}

// Token embedding: out[t, :] = table[ids[t], :], written as float32 (the residual stream is
// held in 32-bit).  An id outside [0, vocab) writes a zero row and records the first such
// token in `status` ({code, token index}); nothing traps.  The reference does the same gather
// with one element per thread and a blocking read of its error flag (src/layers/embedding.cu:91-158).
// A negative id -1-j stands for feedback[j]: the token that the previous step sampled into a
// device buffer, which the host has not read yet when it launches this step.
//
// Also here: the small scatter that applies a step's block-table changes on the device.
#include "common.cuh"

template <typename T>
__global__ void embedding_gather_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab,
                                        int32_t* __restrict__ status, const int32_t* __restrict__ feedback,
                                        int feedback_len, float scale) {
    pdl_begin();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && feedback != nullptr && -1 - id < feedback_len) id = feedback[-1 - id];
    float* o = out + static_cast<size_t>(t) * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && atomicCAS(status, 0, 1) == 0) status[1] = t;
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = 0.0f;
        return;
    }
    const T* row = table + static_cast<size_t>(id) * hidden;
    if ((hidden & 7) == 0) {
        for (int h = threadIdx.x * 8; h < hidden; h += blockDim.x * 8) {
            float v[8];
            load8(row + h, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= scale;      // a design's embedding scale, applied in 32-bit (1: exact)
            store8(o + h, v);
        }
    } else {
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = to_f32(row[h]) * scale;
    }
}

extern "C" int llm_embedding_gather(const int32_t* ids, const void* table, int table_dtype, float* out,
                                    int num_tokens, int hidden, int vocab, int32_t* status,
                                    const int32_t* feedback, int feedback_len, float scale, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (hidden <= 0 || vocab <= 0) return LLM_REFUSED_SIZE;
    if ((hidden & 7) == 0 && (!aligned16(table) || !aligned16(out))) return LLM_REFUSED_ALIGN;
    const int threads = hidden >= 2048 ? 256 : 128;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (table_dtype == LLM_DT_F32)
        launch_pdl((embedding_gather_kernel<float>), dim3(num_tokens), dim3(threads), 0, s, 
            ids, static_cast<const float*>(table), out, hidden, vocab, status, feedback, feedback_len, scale);
    else if (table_dtype == LLM_DT_BF16)
        launch_pdl((embedding_gather_kernel<bf16>), dim3(num_tokens), dim3(threads), 0, s, 
            ids, static_cast<const bf16*>(table), out, hidden, vocab, status, feedback, feedback_len, scale);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

// The same gather for designs that add a sinusoidal position vector to the token's row:
//     out[t, 2i] = table[id, 2i] + sin(p * f_i),  out[t, 2i+1] = table[id, 2i+1] + cos(p * f_i)
// with p the token's position and f_i = inv_freq[i] (a table in double precision made by the host, so
// that the angle p * f_i is exact to the last bit of a float at any position).  The sum is 32-bit.
// `copy` (optional) receives the same row in the compute dtype, for a first layer whose sublayers
// read the stream itself instead of a norm of it.
template <typename T, typename TC>
__global__ void embedding_sinusoid_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                          float* __restrict__ out, TC* __restrict__ copy, int hidden, int vocab,
                                          int32_t* __restrict__ status, const int32_t* __restrict__ feedback,
                                          int feedback_len, const int32_t* __restrict__ positions,
                                          const double* __restrict__ inv_freq) {
    pdl_begin();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && feedback != nullptr && -1 - id < feedback_len) id = feedback[-1 - id];
    float* o = out + static_cast<size_t>(t) * hidden;
    TC* c = copy ? copy + static_cast<size_t>(t) * hidden : nullptr;
    const bool bad = id < 0 || id >= vocab;
    if (bad && threadIdx.x == 0 && atomicCAS(status, 0, 1) == 0) status[1] = t;
    const T* row = table + static_cast<size_t>(bad ? 0 : id) * hidden;
    const double p = static_cast<double>(positions[t]);
    for (int i = threadIdx.x; 2 * i < hidden; i += blockDim.x) {
        double sn, cs;
        sincos(p * inv_freq[i], &sn, &cs);
        const float a = (bad ? 0.0f : to_f32(row[2 * i])) + static_cast<float>(sn);
        o[2 * i] = a;
        if (c) c[2 * i] = from_f32<TC>(a);
        if (2 * i + 1 < hidden) {
            const float b = (bad ? 0.0f : to_f32(row[2 * i + 1])) + static_cast<float>(cs);
            o[2 * i + 1] = b;
            if (c) c[2 * i + 1] = from_f32<TC>(b);
        }
    }
}

extern "C" int llm_embedding_sinusoid(const int32_t* ids, const void* table, int table_dtype, float* out, void* copy,
                                      int copy_dtype, int num_tokens, int hidden, int vocab, int32_t* status,
                                      const int32_t* feedback, int feedback_len, const int32_t* positions,
                                      const double* inv_freq, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (hidden <= 0 || vocab <= 0) return LLM_REFUSED_SIZE;
    const int threads = hidden >= 2048 ? 256 : 128;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define LAUNCH(T, TC)                                                                                          \
    launch_pdl((embedding_sinusoid_kernel<T, TC>), dim3(num_tokens), dim3(threads), 0, s, ids,                 \
               static_cast<const T*>(table), out, static_cast<TC*>(copy), hidden, vocab, status, feedback,     \
               feedback_len, positions, inv_freq)
    if (!copy) copy_dtype = LLM_DT_F32;
    if (table_dtype == LLM_DT_F32 && copy_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (table_dtype == LLM_DT_F32 && copy_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (table_dtype == LLM_DT_BF16 && copy_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else if (table_dtype == LLM_DT_BF16 && copy_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

// dst[index[i]] = value[i] for i < *count (count lives on the device so that a captured
// graph can replay with a different number of updates; a null count means max_count).  An index outside [0, dst_len)
// is skipped and recorded in status.
__global__ void scatter_int32_kernel(int32_t* __restrict__ dst, long long dst_len,
                                     const int32_t* __restrict__ index, const int32_t* __restrict__ value,
                                     const int32_t* __restrict__ count, int max_count,
                                     int32_t* __restrict__ status) {
    // No early invitation here: kernels later in the step read the tables before their own
    // griddepcontrol.wait (they only wait for the kernel just before them), which is safe
    // because nothing after this kernel starts until it has finished.
    pdl_wait();
    const int n = count ? min(*count, max_count) : max_count;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const long long at = index[i];
        if (at < 0 || at >= dst_len) {
            if (atomicCAS(status, 0, 2) == 0) status[1] = i;
            continue;
        }
        dst[at] = value[i];
    }
}

extern "C" int llm_scatter_int32(int32_t* dst, long long dst_len, const int32_t* index,
                                 const int32_t* value, const int32_t* count, int max_count,
                                 int32_t* status, uintptr_t stream) {
    if (max_count <= 0) return LLM_OK;
    const int threads = 256;
    const int blocks = min((max_count + threads - 1) / threads, 64);
    launch_pdl(scatter_int32_kernel, dim3(blocks), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream), 
        dst, dst_len, index, value, count, max_count, status);
    return launch_status();
}

// Gated linear attention: a per-head state S [D, V] that every token decays per key channel and
// adds an outer product to,
//
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          o_t = S_t^T q_t
//
// with the state, the decays and every product of the recurrence in 32-bit CUDA-core arithmetic (the
// recurrence's operands must not be rounded to 16 bits, so this is no tensor-core kernel; its roofline
// is the float32 FMA rate for prompt portions and the state's bytes for single decoded tokens).
//
// gla_decay_kernel   alpha[t, c] = exp(ln(sigmoid(z)) / tau),  z = w2[c, :] . a[t, :] + b2[c]: the second
//                    half of a low-rank decay projection, kept out of the matrix-product path so that its
//                    input is never rounded.  A block takes 32 tokens x 128 channels and reads its slice
//                    of the (transposed) weights once.
// gla_scan_kernel    one block per (work item, head) walks the item's tokens in order.  Thread (dg, v)
//                    keeps rows dg*R .. dg*R+R-1 of column v of the state in registers; tokens are
//                    staged through shared memory sixteen at a time (no barrier between the tokens of a
//                    batch: each row group leaves its share of o in shared memory).  Epilogue per staged
//                    batch, a warp per token: the row groups' shares are added, then RMS norm of o over V,
//                    weight, output gate silu(g), scale, store in the compute dtype into a column range
//                    of the layer's output buffer.
//                    Three modes make long prompt portions parallel over chunks of tokens:
//                      FULL   state in from the request's slot, outputs, state out to the slot
//                             (single decoded tokens and short portions: one pass)
//                      LOCAL  state in = 0, no outputs; the chunk's own contribution L and its total
//                             decay A = prod alpha go to scratch
//                      OUT    state in from scratch (what gla_chain_kernel put there), outputs only
// gla_step_kernel    the same for entries of ONE token (decode steps): the state streams through, see there.
// gla_chain_kernel   per (long entry, head), over its chunks in order: scratch[c] <- S (the state that
//                    enters chunk c), S <- diag(A_c) S + L_c; at the end the slot's state <- S.
//
// A position's output depends on how a prompt is cut only through the order of 32-bit additions.
#include "common.cuh"

#define GLA_TB 16          // tokens staged at a time
#define GLA_FULL 0
#define GLA_LOCAL 1
#define GLA_OUT 2

#define GLA_DECAY_TOKENS 32       // tokens a block of the decay kernel takes
#define GLA_DECAY_CHANNELS 128    // and channels (one a thread)

// w2t is the second half of the decay projection TRANSPOSED, [rank, channels]: thread c of a block reads
// w2t[j][c] for every j once (neighbouring threads read neighbouring words) and applies it to all of the
// block's tokens, whose inputs a[t][:] sit in shared memory.
__global__ void gla_decay_kernel(const float* __restrict__ proj, long long stride, int a_off, int rank,
                                 const float* __restrict__ w2t, const float* __restrict__ b2, float inv_tau,
                                 float* __restrict__ la, int channels, int num_tokens) {
    pdl_begin();
    extern __shared__ float a[];                    // [GLA_DECAY_TOKENS][rank]
    const int t0 = blockIdx.x * GLA_DECAY_TOKENS;
    const int nt = min(GLA_DECAY_TOKENS, num_tokens - t0);
    for (int idx = threadIdx.x; idx < nt * rank; idx += blockDim.x) {
        const int t = idx / rank, j = idx - t * rank;
        a[idx] = proj[static_cast<size_t>(t0 + t) * stride + a_off + j];
    }
    __syncthreads();
    const int c = blockIdx.y * GLA_DECAY_CHANNELS + threadIdx.x;
    if (c >= channels) return;
    float z[GLA_DECAY_TOKENS];
    const float bias = b2 ? b2[c] : 0.0f;
#pragma unroll
    for (int t = 0; t < GLA_DECAY_TOKENS; ++t) z[t] = bias;
    int j = 0;
    for (; j + 16 <= rank; j += 16) {              // sixteen weights in flight: a decode step's few blocks are bound by
        float w[16];                                // the latency of these loads, not by their bytes
#pragma unroll
        for (int u = 0; u < 16; ++u) w[u] = w2t[static_cast<size_t>(j + u) * channels + c];
#pragma unroll
        for (int u = 0; u < 16; ++u)
#pragma unroll
            for (int t = 0; t < GLA_DECAY_TOKENS; ++t)
                if (t < nt) z[t] += w[u] * a[t * rank + j + u];
    }
    for (; j < rank; ++j) {
        const float w = w2t[static_cast<size_t>(j) * channels + c];
#pragma unroll
        for (int t = 0; t < GLA_DECAY_TOKENS; ++t)
            if (t < nt) z[t] += w * a[t * rank + j];
    }
#pragma unroll
    for (int t = 0; t < GLA_DECAY_TOKENS; ++t)
        if (t < nt) {
            // ln(sigmoid(z)) without overflow on either side
            const float ls = z[t] < 0.0f ? z[t] - log1pf(expf(z[t])) : -log1pf(expf(-z[t]));
            la[static_cast<size_t>(t0 + t) * channels + c] = expf(ls * inv_tau);      // alpha = sigmoid(z)^(1/tau)
        }
}

extern "C" int llm_gla_decay(const float* proj, long long stride, int a_off, int rank, const float* w2t, const float* b2,
                             float tau, float* la, int num_tokens, int channels, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (rank <= 0 || channels <= 0 || !(tau > 0.0f) || rank > 1024) return LLM_REFUSED_SIZE;
    const dim3 grid((num_tokens + GLA_DECAY_TOKENS - 1) / GLA_DECAY_TOKENS,
                    (channels + GLA_DECAY_CHANNELS - 1) / GLA_DECAY_CHANNELS);
    if (grid.y > 65535) return LLM_REFUSED_SIZE;
    launch_pdl(gla_decay_kernel, grid, dim3(GLA_DECAY_CHANNELS), GLA_DECAY_TOKENS * rank * sizeof(float),
               reinterpret_cast<cudaStream_t>(stream), proj, stride, a_off, rank, w2t, b2, 1.0f / tau, la, channels,
               num_tokens);
    return launch_status();
}

__device__ __forceinline__ void gla_cp16(float* smem_dst, const float* src) {
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}

// items: int32 [n, 4] = (entry, first row in the batch, tokens, index of the item's scratch) or null: item i
// is entry i, all of it.  `alpha` [T, H*D] are the decays themselves (what gla_decay_kernel writes).
template <int R, int MAX_THREADS, typename TO>
__global__ void __launch_bounds__(MAX_THREADS) gla_scan_kernel(
    const float* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, int g_off,
    const float* __restrict__ alpha, const float* __restrict__ norm_w, float eps, float q_scale, float out_scale,
    TO* __restrict__ out, long long out_stride, int out_off, float* __restrict__ state,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start,
    const int32_t* __restrict__ entry_q_len, const int32_t* __restrict__ items, int mode,
    float* __restrict__ scratch_s, float* __restrict__ scratch_a, int H, int D, int V, int DG, int vec) {
    pdl_begin();
    extern __shared__ __align__(16) float smem[];
    const int h = blockIdx.y;
    int entry, row0, count, sidx;
    if (items) {
        entry = items[4 * blockIdx.x];
        if (entry < 0) return;                       // padding of a work list
        row0 = items[4 * blockIdx.x + 1];
        count = items[4 * blockIdx.x + 2];
        sidx = items[4 * blockIdx.x + 3];
    } else {
        entry = blockIdx.x;
        row0 = entry_q_start[entry];
        count = entry_q_len[entry];
        sidx = entry;
    }
    const int tid = threadIdx.x, nthreads = blockDim.x;
    // thread (dg, v) for tid < V * DG; the block is rounded up to whole warps and the rest only help to stage
    const bool active = tid < V * DG;
    const int v = active ? tid % V : 0, dg = active ? tid / V : 0;
    // two staging buffers of [TB][D] queries, keys, decays and [TB][V] values: batch b+1 is copied in
    // (cp.async, sixteen bytes at a time) while batch b is worked on
    const int buf_floats = GLA_TB * (3 * D + V);
    float* part = smem + 2 * buf_floats;            // [TB][DG][V]: each row group's share of o, added up in the epilogue
    const size_t HD = static_cast<size_t>(H) * D;
    const bool outputs = mode != GLA_LOCAL;
    // a thread whose R rows all exist reads its decays, keys and queries sixteen bytes at a time
    const bool whole = active && dg * R + R <= D && (D & 3) == 0;

    float S[R];
    float* slot_state = state + (static_cast<size_t>(entry_slot[entry]) * H + h) * D * V;
    const float* s_in = mode == GLA_FULL ? slot_state
                        : (mode == GLA_OUT ? scratch_s + (static_cast<size_t>(sidx) * H + h) * D * V : nullptr);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = dg * R + r;
        S[r] = (s_in && active && d < D) ? s_in[static_cast<size_t>(d) * V + v] : 0.0f;
    }

    auto stage = [&](int done, int buf) {
        const int nb = min(GLA_TB, count - done);
        const size_t base = static_cast<size_t>(row0 + done);
        float* bq = smem + buf * buf_floats;
        float* bk = bq + GLA_TB * D;
        float* ba = bk + GLA_TB * D;
        float* bv = ba + GLA_TB * D;
        if (vec) {
            const int d4 = D >> 2, v4 = V >> 2;
            for (int idx = tid; idx < nb * d4; idx += nthreads) {
                const int tok = idx / d4, c = (idx - tok * d4) << 2;
                const float* pr = proj + (base + tok) * stride + h * D + c;
                gla_cp16(bk + tok * D + c, pr + k_off);
                gla_cp16(ba + tok * D + c, alpha + (base + tok) * HD + h * D + c);
                if (outputs) gla_cp16(bq + tok * D + c, pr + q_off);
            }
            for (int idx = tid; idx < nb * v4; idx += nthreads) {
                const int tok = idx / v4, c = (idx - tok * v4) << 2;
                gla_cp16(bv + tok * V + c, proj + (base + tok) * stride + v_off + h * V + c);
            }
            asm volatile("cp.async.commit_group;\n" ::);
        } else {
            for (int idx = tid; idx < nb * D; idx += nthreads) {
                const int tok = idx / D, d = idx - tok * D;
                const float* pr = proj + (base + tok) * stride + h * D + d;
                bk[idx] = pr[k_off];
                ba[idx] = alpha[(base + tok) * HD + h * D + d];
                if (outputs) bq[idx] = pr[q_off];
            }
            for (int idx = tid; idx < nb * V; idx += nthreads) {
                const int tok = idx / V, c = idx - tok * V;
                bv[idx] = proj[(base + tok) * stride + v_off + h * V + c];
            }
        }
    };

    stage(0, 0);
    for (int done = 0, b = 0; done < count; done += GLA_TB, ++b) {
        const int nb = min(GLA_TB, count - done);
        const size_t base = static_cast<size_t>(row0 + done);
        const bool more = done + GLA_TB < count;
        if (more) stage(done + GLA_TB, (b + 1) & 1);
        if (vec) {
            if (more) asm volatile("cp.async.wait_group 1;\n" ::: "memory");
            else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* sq = smem + (b & 1) * buf_floats;
        const float* sk = sq + GLA_TB * D;
        const float* sa = sk + GLA_TB * D;
        const float* sv = sa + GLA_TB * D;
        for (int tok = 0; tok < nb; ++tok) {
            const float vt = sv[tok * V + v];
            const float* a = sa + tok * D + dg * R;
            const float* k = sk + tok * D + dg * R;
            const float* q = sq + tok * D + dg * R;
            float p0 = 0.0f, p1 = 0.0f;
            if (whole) {
                const float4* a4 = reinterpret_cast<const float4*>(a);
                const float4* k4 = reinterpret_cast<const float4*>(k);
                const float4* q4 = reinterpret_cast<const float4*>(q);
                if (outputs) {
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        const float4 av = a4[r >> 2], kv = k4[r >> 2], qv = q4[r >> 2];
                        S[r] = av.x * S[r] + kv.x * vt;             p0 += S[r] * qv.x;
                        S[r + 1] = av.y * S[r + 1] + kv.y * vt;     p1 += S[r + 1] * qv.y;
                        S[r + 2] = av.z * S[r + 2] + kv.z * vt;     p0 += S[r + 2] * qv.z;
                        S[r + 3] = av.w * S[r + 3] + kv.w * vt;     p1 += S[r + 3] * qv.w;
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        const float4 av = a4[r >> 2], kv = k4[r >> 2];
                        S[r] = av.x * S[r] + kv.x * vt;
                        S[r + 1] = av.y * S[r + 1] + kv.y * vt;
                        S[r + 2] = av.z * S[r + 2] + kv.z * vt;
                        S[r + 3] = av.w * S[r + 3] + kv.w * vt;
                    }
                }
            } else if (active) {
#pragma unroll
                for (int r = 0; r < R; r += 2) {
                    if (dg * R + r < D) {
                        S[r] = a[r] * S[r] + k[r] * vt;
                        if (outputs) p0 += S[r] * q[r];
                    }
                    if (dg * R + r + 1 < D) {
                        S[r + 1] = a[r + 1] * S[r + 1] + k[r + 1] * vt;
                        if (outputs) p1 += S[r + 1] * q[r + 1];
                    }
                }
            }
            if (outputs && active) part[(tok * DG + dg) * V + v] = p0 + p1;
        }
        __syncthreads();
        if (outputs) {                              // a warp per token: add the row groups, norm over V, weight, gate, scale
            const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
            for (int tok = warp; tok < nb; tok += nwarps) {
                float* o = part + tok * DG * V;
                float ss = 0.0f;
                for (int c = lane; c < V; c += 32) {
                    float sum = o[c];
                    for (int g2 = 1; g2 < DG; ++g2) sum += o[g2 * V + c];
                    sum *= q_scale;                 // q = W_q x * q_scale, applied to the finished sum
                    o[c] = sum;
                    ss += sum * sum;
                }
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / static_cast<float>(V) + eps);
                const float* gr = proj + (base + tok) * stride + g_off + h * V;
                TO* orow = out + (base + tok) * out_stride + out_off + h * V;
                for (int c = lane; c < V; c += 32) {
                    const float g = gr[c];
                    const float silu = g / (1.0f + expf(-g));
                    orow[c] = from_f32<TO>(o[c] * inv * norm_w[c] * silu * out_scale);
                }
            }
        }
        __syncthreads();                            // this buffer is filled again two batches on
    }
    if (mode == GLA_OUT) return;
    float* s_out = mode == GLA_FULL ? slot_state : scratch_s + (static_cast<size_t>(sidx) * H + h) * D * V;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = dg * R + r;
        if (active && d < D) s_out[static_cast<size_t>(d) * V + v] = S[r];
    }
    if (mode == GLA_LOCAL) {                        // the chunk's total decay per key channel
        for (int d = tid; d < D; d += nthreads) {
            float prod = 1.0f;
            for (int tok = 0; tok < count; ++tok) prod *= alpha[(static_cast<size_t>(row0) + tok) * HD + h * D + d];
            scratch_a[(static_cast<size_t>(sidx) * H + h) * D + d] = prod;
        }
    }
}

// Rows of a state column that one thread keeps (R), the row groups DG = ceil(D / R), and the block size the
// kernel is compiled for: 16, else 32, else 64, else 8 rows, whichever block of V * DG threads fits first
// within 512 threads (64 x 64 a head: 110 us with 16 rows, 134 with 8, 173 with 32 for 2,048 tokens of 16
// heads; 128 x 128: 32 rows, 185 us for 8 heads), then within what the kernel's registers allow at that R (a block's registers are threads x registers
// per thread, at most 65,536).  States too large for that (128 x 256 a head and more) take R = 64 compiled
// for 512 or 1,024 threads: the compiler then keeps part of the state in local memory, which is slow and
// correct.
static int gla_rows_per_thread(int D, int V, int* dg_out, int* max_threads) {
    const int cands[4] = {8, 16, 32, 64};
    const int limits[2][4] = {{512, 512, 512, 384}, {1024, 1024, 512, 384}};
    const int compiled_for[4] = {1024, 1024, 512, 384};
    static int forced = -1;                        // LLM_GLA_ROWS=8|16|32|64: take that R when its block fits (for measurements)
    if (forced < 0) {
        const char* e = getenv("LLM_GLA_ROWS");
        forced = e ? atoi(e) : 0;
    }
    for (int c = 0; c < 4; ++c)
        if (forced == cands[c] && static_cast<long long>(V) * ((D + forced - 1) / forced) <= limits[1][c]) {
            *dg_out = (D + forced - 1) / forced;
            *max_threads = compiled_for[c];
            return forced;
        }
    const int order[4] = {1, 2, 3, 0};             // 16 rows a thread first: measured best wherever its block fits 512 threads
    for (int pass = 0; pass < 2; ++pass)
        for (int o = 0; o < 4; ++o) {
            const int c = order[o];
            const int dg = (D + cands[c] - 1) / cands[c];
            if (static_cast<long long>(V) * dg <= limits[pass][c]) {
                *dg_out = dg;
                *max_threads = compiled_for[c];
                return cands[c];
            }
        }
    const int dg = (D + 63) / 64;
    for (int limit = 512; limit <= 1024; limit *= 2)
        if (static_cast<long long>(V) * dg <= limit) {
            *dg_out = dg;
            *max_threads = limit;
            return 64;
        }
    return 0;
}

extern "C" int llm_gla_supported(int D, int V) {
    int dg, mt;
    return (D > 0 && V > 0 && gla_rows_per_thread(D, V, &dg, &mt) > 0) ? 1 : 0;
}

extern "C" int llm_gla_scan(
    const float* proj, long long stride, int q_off, int k_off, int v_off, int g_off, const float* la,
    const float* norm_w, float eps, float q_scale, float out_scale, void* out, int out_dtype, long long out_stride,
    int out_off, float* state, const int32_t* entry_slot, const int32_t* entry_q_start, const int32_t* entry_q_len,
    const int32_t* items, int num_items, int mode, float* scratch_s, float* scratch_a, int H, int D, int V,
    uintptr_t stream) {
    if (num_items <= 0) return LLM_OK;
    if (H <= 0 || D <= 0 || V <= 0 || mode < 0 || mode > 2 || H > 65535) return LLM_REFUSED_SIZE;
    if (mode != GLA_FULL && (!items || !scratch_s || !scratch_a)) return LLM_REFUSED_SIZE;
    int DG = 0, MT = 0;
    const int R = gla_rows_per_thread(D, V, &DG, &MT);
    if (R == 0) return LLM_REFUSED_SIZE;
    const size_t smem = static_cast<size_t>(GLA_TB) * (2 * (3 * D + V) + static_cast<size_t>(DG) * V) * sizeof(float);
    // sixteen-byte copies into the staging buffers want every row piece on a sixteen-byte boundary
    const int vec = D % 4 == 0 && V % 4 == 0 && stride % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                    aligned16(proj) && aligned16(la);
    if (smem > 220 * 1024) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(num_items, H), block((V * DG + 31) / 32 * 32);
#define LAUNCH(RR, MM, TO)                                                                                        \
    do {                                                                                                          \
        auto kern = gla_scan_kernel<RR, MM, TO>;                                                                    \
        if (smem > 48 * 1024) {                                                                                   \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                                       static_cast<int>(smem));                                   \
            if (e != cudaSuccess) return static_cast<int>(e);                                                     \
        }                                                                                                         \
        launch_pdl(kern, grid, block, smem, s, proj, stride, q_off, k_off, v_off, g_off, la, norm_w, eps, q_scale, \
                   out_scale, static_cast<TO*>(out), out_stride, out_off, state, entry_slot, entry_q_start,       \
                   entry_q_len, items, mode, scratch_s, scratch_a, H, D, V, DG, vec);                             \
    } while (0)
#define BY_R(TO)                                                                                                  \
    switch (R) {                                                                                                  \
        case 8: LAUNCH(8, 1024, TO); break;                                                                       \
        case 16: LAUNCH(16, 1024, TO); break;                                                                     \
        case 32: LAUNCH(32, 512, TO); break;                                                                      \
        default:                                                                                                  \
            if (MT == 384) LAUNCH(64, 384, TO);                                                                   \
            else if (MT == 512) LAUNCH(64, 512, TO);                                                              \
            else LAUNCH(64, 1024, TO);                                                                            \
            break;                                                                                                \
    }
    if (out_dtype == LLM_DT_F32) { BY_R(float) }
    else if (out_dtype == LLM_DT_BF16) { BY_R(bf16) }
    else return LLM_REFUSED_DTYPE;
#undef BY_R
#undef LAUNCH
    return launch_status();
}

// The recurrence for entries that bring ONE token (decode steps): the state is streamed, not held: thread
// (row group, column) walks its rows of the column once, eight loads in flight, S <- alpha S + k v written
// back as it goes, its share of o left in shared memory; then a warp per 32 columns adds the shares and
// applies norm, weight, gate and scale.  Few registers, so several blocks share an SM and the state's
// bytes bound the kernel, as keys and values bound decode attention.  Entry i is row q_start[i].
template <typename TO>
__global__ void gla_step_kernel(
    const float* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, int g_off,
    const float* __restrict__ la, const float* __restrict__ norm_w, float eps, float q_scale, float out_scale,
    TO* __restrict__ out, long long out_stride, int out_off, float* __restrict__ state,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start, int H, int D, int V, int DG,
    int a_off, int rank, const float* __restrict__ w2t, const float* __restrict__ b2, float inv_tau) {
    pdl_begin();
    extern __shared__ __align__(16) float smem[];
    float* sq = smem;                 // [D]
    float* sk = sq + D;
    float* sa = sk + D;
    float* sv = sa + D;               // [V]
    float* part = sv + V;             // [DG][V]
    float* red = part + DG * V;       // 33
    float* a1 = red + 33;             // [rank]: the decay projection's first half, when the decays are made here
    const int entry = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const size_t row = static_cast<size_t>(entry_q_start[entry]);
    const float* pr = proj + row * stride;
    if (!la) {
        for (int j = tid; j < rank; j += blockDim.x) a1[j] = pr[a_off + j];
        __syncthreads();
    }
    for (int d = tid; d < D; d += blockDim.x) {
        sq[d] = pr[q_off + h * D + d] * q_scale;
        sk[d] = pr[k_off + h * D + d];
        if (la) {
            sa[d] = la[row * H * D + h * D + d];       // the decay itself
        } else {                                       // alpha = sigmoid(w2[c, :] . a1 + b2[c]) ^ (1 / tau), as gla_decay_kernel
            const int c = h * D + d, C = H * D;
            float z = b2 ? b2[c] : 0.0f;
            int j = 0;
            for (; j + 16 <= rank; j += 16) {
                float w[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) w[u] = w2t[static_cast<size_t>(j + u) * C + c];
#pragma unroll
                for (int u = 0; u < 16; ++u) z += w[u] * a1[j + u];
            }
            for (; j < rank; ++j) z += w2t[static_cast<size_t>(j) * C + c] * a1[j];
            const float ls = z < 0.0f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
            sa[d] = expf(ls * inv_tau);
        }
    }
    for (int c = tid; c < V; c += blockDim.x) sv[c] = pr[v_off + h * V + c];
    __syncthreads();
    const bool active = tid < V * DG;
    const int c = active ? tid % V : 0, dg = active ? tid / V : 0;
    const int rows = (D + DG - 1) / DG, d0 = dg * rows, d1 = min(D, d0 + rows);
    float* S = state + (static_cast<size_t>(entry_slot[entry]) * H + h) * D * V + c;
    if (active) {
        const float vt = sv[c];
        float p = 0.0f;
        int d = d0;
        for (; d + 8 <= d1; d += 8) {
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = S[static_cast<size_t>(d + u) * V];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                x[u] = sa[d + u] * x[u] + sk[d + u] * vt;
                S[static_cast<size_t>(d + u) * V] = x[u];
                p += x[u] * sq[d + u];
            }
        }
        for (; d < d1; ++d) {
            const float x = sa[d] * S[static_cast<size_t>(d) * V] + sk[d] * vt;
            S[static_cast<size_t>(d) * V] = x;
            p += x * sq[d];
        }
        part[dg * V + c] = p;
    }
    __syncthreads();
    float ss = 0.0f;
    for (int i = tid; i < V; i += blockDim.x) {
        float o = part[i];
        for (int g2 = 1; g2 < DG; ++g2) o += part[g2 * V + i];
        part[i] = o;
        ss += o * o;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(V) + eps);
    TO* orow = out + row * out_stride + out_off + h * V;
    for (int i = tid; i < V; i += blockDim.x) {
        const float g = pr[g_off + h * V + i];
        orow[i] = from_f32<TO>(part[i] * inv * norm_w[i] * (g / (1.0f + expf(-g))) * out_scale);
    }
}

extern "C" int llm_gla_step(
    const float* proj, long long stride, int q_off, int k_off, int v_off, int g_off, const float* la,
    const float* norm_w, float eps, float q_scale, float out_scale, void* out, int out_dtype, long long out_stride,
    int out_off, float* state, const int32_t* entry_slot, const int32_t* entry_q_start, int num_entries, int H, int D,
    int V, int a_off, int rank, const float* w2t, const float* b2, float tau, uintptr_t stream) {
    // la null: the decays are computed here from the projection's columns a_off .. a_off + rank (w2t, b2, tau as
    // for llm_gla_decay), which saves a decode step one launch a layer
    if (num_entries <= 0) return LLM_OK;
    if (H <= 0 || D <= 0 || V <= 0 || H > 65535 || V > 1024) return LLM_REFUSED_SIZE;
    if (!la && (!w2t || rank <= 0 || rank > 4096 || !(tau > 0.0f))) return LLM_REFUSED_SIZE;
    if (la) rank = 0;
    int DG = 256 / V;
    if (DG < 1) DG = 1;
    if (DG > D) DG = D;
    const int threads = (V * DG + 31) / 32 * 32;
    const size_t smem = (3 * static_cast<size_t>(D) + V + static_cast<size_t>(DG) * V + 33 + rank) * sizeof(float);
    if (smem > 48 * 1024) return LLM_REFUSED_SIZE;
    const float inv_tau = la ? 0.0f : 1.0f / tau;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(num_entries, H);
    if (out_dtype == LLM_DT_F32)
        launch_pdl((gla_step_kernel<float>), grid, dim3(threads), smem, s, proj, stride, q_off, k_off, v_off, g_off, la, norm_w,
                   eps, q_scale, out_scale, static_cast<float*>(out), out_stride, out_off, state, entry_slot, entry_q_start,
                   H, D, V, DG, a_off, rank, w2t, b2, inv_tau);
    else if (out_dtype == LLM_DT_BF16)
        launch_pdl((gla_step_kernel<bf16>), grid, dim3(threads), smem, s, proj, stride, q_off, k_off, v_off, g_off, la, norm_w,
                   eps, q_scale, out_scale, static_cast<bf16*>(out), out_stride, out_off, state, entry_slot, entry_q_start,
                   H, D, V, DG, a_off, rank, w2t, b2, inv_tau);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

// chains: int32 [n, 3] = (entry, first scratch index, number of chunks); chunk c of the entry is scratch
// index first + c.  grid (n, H, blocks over D*V).
__global__ void gla_chain_kernel(float* __restrict__ state, float* __restrict__ scratch_s,
                                 const float* __restrict__ scratch_a, const int32_t* __restrict__ chains,
                                 const int32_t* __restrict__ entry_slot, int H, int D, int V) {
    pdl_begin();
    const int entry = chains[3 * blockIdx.x];
    if (entry < 0) return;
    const int first = chains[3 * blockIdx.x + 1], n = chains[3 * blockIdx.x + 2];
    const int h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= D * V) return;
    const int d = e / V;
    float* st = state + (static_cast<size_t>(entry_slot[entry]) * H + h) * D * V + e;
    float S = *st;
    for (int c0 = 0; c0 < n; c0 += 8) {              // eight chunks' loads in flight, then the chain through them
        float L[8], A[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const size_t at = static_cast<size_t>(first + min(c0 + i, n - 1)) * H + h;
            L[i] = scratch_s[at * D * V + e];
            A[i] = scratch_a[at * D + d];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c0 + i < n) {
                scratch_s[(static_cast<size_t>(first + c0 + i) * H + h) * D * V + e] = S;
                S = A[i] * S + L[i];
            }
    }
    *st = S;
}

extern "C" int llm_gla_chain(float* state, float* scratch_s, const float* scratch_a, const int32_t* chains,
                             int num_chains, const int32_t* entry_slot, int H, int D, int V, uintptr_t stream) {
    if (num_chains <= 0) return LLM_OK;
    if (H <= 0 || D <= 0 || V <= 0 || H > 65535) return LLM_REFUSED_SIZE;
    const int threads = 256;
    const int bz = (D * V + threads - 1) / threads;
    if (bz > 65535) return LLM_REFUSED_SIZE;
    launch_pdl(gla_chain_kernel, dim3(num_chains, H, bz), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
               state, scratch_s, scratch_a, chains, entry_slot, H, D, V);
    return launch_status();
}

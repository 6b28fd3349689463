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
//
// The same kernels run every recurrence of that shape whose decay is one number per (token, head) or a
// constant per head (template SCALAR of the scan kernel; strides of `alpha` in the step kernel):
//
//     S_t = a_t S_(t-1) + e_t k_t v_t^T     [ n_t = a_t n_(t-1) + e_t k_t ]      o_t = S_t^T q_t [ / den_t ]
//
// with an optional input scale e per (token, head) and an optional normaliser vector n kept beside S (an
// extra column of the state whose "value" is 1): den_t = max(|n_t . q_t|, floor_t) + 1e-6 with a floor per
// (token, head).  Retention: a = a constant per head, no e, no n.  A matrix memory with exponential
// gates: a, e and floor come from recur_gates_kernel (prompt portions) or are made inside the step
// kernel (decode steps).  The epilogue's output norm takes a weight [V] shared by the heads, a weight
// per head, or none, and its gate is silu or a sigmoid.  A head's state in a slot is S [D, V], then
// n [D] when there is one, then whatever else the mixer keeps there (`state_head_stride`).
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
// What varies between the recurrences that share these kernels (see the top of the file).
struct RecurOpts {
    long long a_tok, a_head;          // SCALAR: alpha index = token * a_tok + head * a_head
    const float* kscale;              // SCALAR: e per (token, head) at token * H + head, or null
    const float* nfloor;              // floor per (token, head): non-null means the state has a normaliser column
    int norm_stride;                  // output norm weight index = head * norm_stride + channel (0: shared by the heads)
    int gate_kind;                    // 0 none, 1 sigmoid, 2 silu
    long long state_head_stride, state_slot_stride;
};

__device__ __forceinline__ float recur_gate(float g, int kind) {
    if (kind == 0) return 1.0f;
    const float sg = 1.0f / (1.0f + expf(-g));
    return kind == 1 ? sg : g * sg;
}

template <int R, int MAX_THREADS, typename TO, bool SCALAR>
__global__ void __launch_bounds__(MAX_THREADS) gla_scan_kernel(
    const float* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, int g_off,
    const float* __restrict__ alpha, const float* __restrict__ norm_w, float eps, float q_scale, float out_scale,
    TO* __restrict__ out, long long out_stride, int out_off, float* __restrict__ state,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start,
    const int32_t* __restrict__ entry_q_len, const int32_t* __restrict__ items, int mode,
    float* __restrict__ scratch_s, float* __restrict__ scratch_a, int H, int D, int V, int DG, int vec,
    const RecurOpts opt) {
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
    // thread (dg, v) for tid < VC * DG; the block is rounded up to whole warps and the rest only help to stage.
    // Column V (when there is one) is the normaliser n, whose "value" is 1.
    // (what only the SCALAR recurrences use folds away in the per-channel instantiation, whose register budget is tight)
    const float* nfloor = SCALAR ? opt.nfloor : nullptr;
    const int norm_stride = SCALAR ? opt.norm_stride : 0;
    const int gate_kind = SCALAR ? opt.gate_kind : 2;
    const long long head_stride = SCALAR ? opt.state_head_stride : static_cast<long long>(D) * V;
    const long long slot_stride = SCALAR ? opt.state_slot_stride : static_cast<long long>(H) * D * V;
    const int VC = V + (nfloor ? 1 : 0);
    const bool active = tid < VC * DG;
    const int v = active ? tid % VC : 0, dg = active ? tid / VC : 0;
    // two staging buffers of [TB][D] queries, keys, decays and [TB][V] values ([TB] decays and [TB] input
    // scales instead of [TB][D] decays when SCALAR): batch b+1 is copied in (cp.async, sixteen bytes at a
    // time) while batch b is worked on
    const int buf_floats = SCALAR ? GLA_TB * (2 * D + V + 2) : GLA_TB * (3 * D + V);
    float* part = smem + 2 * buf_floats;            // [TB][DG][VC]: each row group's share of o, added up in the epilogue
    const size_t HD = static_cast<size_t>(H) * D;
    const bool outputs = mode != GLA_LOCAL;
    // a thread whose R rows all exist reads its decays, keys and queries sixteen bytes at a time
    const bool whole = active && dg * R + R <= D && (D & 3) == 0;

    float S[R];
    float* slot_state = state + static_cast<size_t>(entry_slot[entry]) * slot_stride + h * head_stride;
    const size_t chunk_state = static_cast<size_t>(D) * VC;     // a chunk's scratch holds S and n, nothing else
    const float* s_in = mode == GLA_FULL ? slot_state
                        : (mode == GLA_OUT ? scratch_s + (static_cast<size_t>(sidx) * H + h) * chunk_state : nullptr);
    // element (d, v) of a head's state: S[d][v] for v < V, then n[d]
    auto at = [&](int d) { return v < V ? static_cast<size_t>(d) * V + v : static_cast<size_t>(D) * V + d; };
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = dg * R + r;
        S[r] = (s_in && active && d < D) ? s_in[at(d)] : 0.0f;
    }

    auto stage = [&](int done, int buf) {
        const int nb = min(GLA_TB, count - done);
        const size_t base = static_cast<size_t>(row0 + done);
        float* bq = smem + buf * buf_floats;
        float* bk = bq + GLA_TB * D;
        float* ba = bk + GLA_TB * D;
        float* bv = SCALAR ? ba : ba + GLA_TB * D;
        if (SCALAR) {                                // the batch's decays and input scales: two numbers a token
            float* bs = bv + GLA_TB * V;
            if (tid < nb) {
                bs[tid] = alpha[(base + tid) * opt.a_tok + h * opt.a_head];
                bs[GLA_TB + tid] = opt.kscale ? opt.kscale[(base + tid) * H + h] : 1.0f;
            }
        }
        if (vec) {
            const int d4 = D >> 2, v4 = V >> 2;
            for (int idx = tid; idx < nb * d4; idx += nthreads) {
                const int tok = idx / d4, c = (idx - tok * d4) << 2;
                const float* pr = proj + (base + tok) * stride + h * D + c;
                gla_cp16(bk + tok * D + c, pr + k_off);
                if (!SCALAR) gla_cp16(ba + tok * D + c, alpha + (base + tok) * HD + h * D + c);
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
                if (!SCALAR) ba[idx] = alpha[(base + tok) * HD + h * D + d];
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
        const float* sv = SCALAR ? sa : sa + GLA_TB * D;
        const float* ss2 = sv + GLA_TB * V;         // SCALAR: [TB] decays, [TB] input scales
        for (int tok = 0; tok < nb; ++tok) {
            float vt = v < V ? sv[tok * V + v] : 1.0f;
            const float* a = sa + tok * D + dg * R;
            const float* k = sk + tok * D + dg * R;
            const float* q = sq + tok * D + dg * R;
            float p0 = 0.0f, p1 = 0.0f;
            if (SCALAR) {
                const float a1 = ss2[tok];
                vt *= ss2[GLA_TB + tok];
                if (whole) {
                    const float4* k4 = reinterpret_cast<const float4*>(k);
                    const float4* q4 = reinterpret_cast<const float4*>(q);
#pragma unroll
                    for (int r = 0; r < R; r += 4) {
                        const float4 kv = k4[r >> 2];
                        S[r] = a1 * S[r] + kv.x * vt;
                        S[r + 1] = a1 * S[r + 1] + kv.y * vt;
                        S[r + 2] = a1 * S[r + 2] + kv.z * vt;
                        S[r + 3] = a1 * S[r + 3] + kv.w * vt;
                        if (outputs) {
                            const float4 qv = q4[r >> 2];
                            p0 += S[r] * qv.x;
                            p1 += S[r + 1] * qv.y;
                            p0 += S[r + 2] * qv.z;
                            p1 += S[r + 3] * qv.w;
                        }
                    }
                } else if (active) {
#pragma unroll
                    for (int r = 0; r < R; ++r)
                        if (dg * R + r < D) {
                            S[r] = a1 * S[r] + k[r] * vt;
                            if (outputs) p0 += S[r] * q[r];
                        }
                }
            } else if (whole) {
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
            if (outputs && active) part[(tok * DG + dg) * VC + v] = p0 + p1;
        }
        __syncthreads();
        if (outputs) {                              // a warp per token: add the row groups, norm over V, weight, gate, scale
            const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
            for (int tok = warp; tok < nb; tok += nwarps) {
                float* o = part + tok * DG * VC;
                float mul = q_scale;                // q = W_q x * q_scale, applied to the finished sum
                if (nfloor) {                       // the normaliser: n . q, floored, divides the output
                    float nq = o[V];
                    for (int g2 = 1; g2 < DG; ++g2) nq += o[g2 * VC + V];
                    nq *= q_scale;
                    mul = q_scale / (fmaxf(fabsf(nq), nfloor[(base + tok) * H + h]) + 1e-6f);
                }
                __syncwarp();
                float ss = 0.0f;
                for (int c = lane; c < V; c += 32) {
                    float sum = o[c];
                    for (int g2 = 1; g2 < DG; ++g2) sum += o[g2 * VC + c];
                    sum *= mul;
                    o[c] = sum;
                    ss += sum * sum;
                }
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / static_cast<float>(V) + eps);
                const float* gr = proj + (base + tok) * stride + g_off + h * V;
                const float* nw = norm_w + h * norm_stride;
                TO* orow = out + (base + tok) * out_stride + out_off + h * V;
                for (int c = lane; c < V; c += 32)
                    orow[c] = from_f32<TO>(o[c] * inv * ((SCALAR && !norm_w) ? 1.0f : nw[c]) * recur_gate(gr[c], gate_kind) * out_scale);
            }
        }
        __syncthreads();                            // this buffer is filled again two batches on
    }
    if (mode == GLA_OUT) return;
    float* s_out = mode == GLA_FULL ? slot_state : scratch_s + (static_cast<size_t>(sidx) * H + h) * chunk_state;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = dg * R + r;
        if (active && d < D) s_out[at(d)] = S[r];
    }
    if (mode == GLA_LOCAL) {                        // the chunk's total decay per key channel
        for (int d = tid; d < D; d += nthreads) {
            float prod = 1.0f;
            for (int tok = 0; tok < count; ++tok)
                prod *= SCALAR ? alpha[(static_cast<size_t>(row0) + tok) * opt.a_tok + h * opt.a_head]
                               : alpha[(static_cast<size_t>(row0) + tok) * HD + h * D + d];
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
// `wide32`: a block of up to 544 threads at 32 rows a thread is allowed (17 warps: a state of 128 x 128 with one
// more column, the normaliser of a matrix memory, is 4 row groups x 129 columns = 516 threads; at 64 rows a
// thread it would run half as fast).
static int gla_rows_per_thread(int D, int V, int* dg_out, int* max_threads, bool wide32 = false) {
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
            if (wide32 && cands[c] == 32 && static_cast<long long>(V) * dg <= 544) {
                *dg_out = dg;
                *max_threads = 544;
                return 32;
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

// The general entry point.  decay_kind 0: a decay per (token, head, key channel), `alpha` [T, H*D]; 1: a decay
// per (token, head) at alpha[token * a_tok + head * a_head] (a_tok 0: a constant per head), with `kscale` and
// `nfloor` as in RecurOpts.  norm_w null: a weightless output norm.
extern "C" int llm_recur_scan(
    const float* proj, long long stride, int q_off, int k_off, int v_off, int g_off, const float* la,
    const float* norm_w, float eps, float q_scale, float out_scale, void* out, int out_dtype, long long out_stride,
    int out_off, float* state, const int32_t* entry_slot, const int32_t* entry_q_start, const int32_t* entry_q_len,
    const int32_t* items, int num_items, int mode, float* scratch_s, float* scratch_a, int H, int D, int V,
    int decay_kind, long long a_tok, long long a_head, const float* kscale, const float* nfloor, int norm_stride,
    int gate_kind, long long state_head_stride, long long state_slot_stride, uintptr_t stream) {
    if (num_items <= 0) return LLM_OK;
    if (H <= 0 || D <= 0 || V <= 0 || mode < 0 || mode > 2 || H > 65535) return LLM_REFUSED_SIZE;
    if (mode != GLA_FULL && (!items || !scratch_s || !scratch_a)) return LLM_REFUSED_SIZE;
    if (decay_kind < 0 || decay_kind > 1 || gate_kind < 0 || gate_kind > 2) return LLM_REFUSED_SIZE;
    // the per-channel instantiation is gated linear attention as it was: its options are fixed
    if (decay_kind == 0 && (kscale || nfloor || !norm_w || norm_stride != 0 || gate_kind != 2 ||
                            state_head_stride != static_cast<long long>(D) * V ||
                            state_slot_stride != static_cast<long long>(H) * D * V))
        return LLM_REFUSED_SIZE;
    const int VC = V + (nfloor ? 1 : 0);
    if (state_head_stride < static_cast<long long>(D) * VC) return LLM_REFUSED_SIZE;
    int DG = 0, MT = 0;
    const int R = gla_rows_per_thread(D, VC, &DG, &MT, decay_kind == 1);
    if (R == 0) return LLM_REFUSED_SIZE;
    const size_t per_buf = decay_kind ? (2 * static_cast<size_t>(D) + V + 2) : (3 * static_cast<size_t>(D) + V);
    const size_t smem = static_cast<size_t>(GLA_TB) * (2 * per_buf + static_cast<size_t>(DG) * VC) * sizeof(float);
    // sixteen-byte copies into the staging buffers want every row piece on a sixteen-byte boundary
    const int vec = D % 4 == 0 && V % 4 == 0 && stride % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                    aligned16(proj) && (decay_kind || aligned16(la));
    if (smem > 220 * 1024) return LLM_REFUSED_SIZE;
    const RecurOpts opt = {a_tok, a_head, kscale, nfloor, norm_stride, gate_kind, state_head_stride, state_slot_stride};
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(num_items, H), block((VC * DG + 31) / 32 * 32);
#define LAUNCH(RR, MM, TO, SC)                                                                                    \
    do {                                                                                                          \
        auto kern = gla_scan_kernel<RR, MM, TO, SC>;                                                                \
        if (smem > 48 * 1024) {                                                                                   \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                                       static_cast<int>(smem));                                   \
            if (e != cudaSuccess) return static_cast<int>(e);                                                     \
        }                                                                                                         \
        launch_pdl(kern, grid, block, smem, s, proj, stride, q_off, k_off, v_off, g_off, la, norm_w, eps, q_scale, \
                   out_scale, static_cast<TO*>(out), out_stride, out_off, state, entry_slot, entry_q_start,       \
                   entry_q_len, items, mode, scratch_s, scratch_a, H, D, V, DG, vec, opt);                        \
    } while (0)
#define BY_R(TO, SC)                                                                                              \
    switch (R) {                                                                                                  \
        case 8: LAUNCH(8, 1024, TO, SC); break;                                                                   \
        case 16: LAUNCH(16, 1024, TO, SC); break;                                                                 \
        case 32: LAUNCH(32, 512, TO, SC); break;                                                                  \
        default:                                                                                                  \
            if (MT == 384) LAUNCH(64, 384, TO, SC);                                                               \
            else if (MT == 512) LAUNCH(64, 512, TO, SC);                                                          \
            else LAUNCH(64, 1024, TO, SC);                                                                        \
            break;                                                                                                \
    }
    if (out_dtype != LLM_DT_F32 && out_dtype != LLM_DT_BF16) return LLM_REFUSED_DTYPE;
    if (R == 32 && MT == 544) {
        if (out_dtype == LLM_DT_F32) LAUNCH(32, 544, float, true);
        else LAUNCH(32, 544, bf16, true);
    } else if (out_dtype == LLM_DT_F32) { if (decay_kind) { BY_R(float, true) } else { BY_R(float, false) } }
    else { if (decay_kind) { BY_R(bf16, true) } else { BY_R(bf16, false) } }
#undef BY_R
#undef LAUNCH
    return launch_status();
}

// Gated linear attention: a decay per key channel, a norm weight [V] shared by the heads, a silu gate, the
// states [slots, H, D, V] alone in their slots.
extern "C" int llm_gla_scan(
    const float* proj, long long stride, int q_off, int k_off, int v_off, int g_off, const float* la,
    const float* norm_w, float eps, float q_scale, float out_scale, void* out, int out_dtype, long long out_stride,
    int out_off, float* state, const int32_t* entry_slot, const int32_t* entry_q_start, const int32_t* entry_q_len,
    const int32_t* items, int num_items, int mode, float* scratch_s, float* scratch_a, int H, int D, int V,
    uintptr_t stream) {
    return llm_recur_scan(proj, stride, q_off, k_off, v_off, g_off, la, norm_w, eps, q_scale, out_scale, out, out_dtype,
                          out_stride, out_off, state, entry_slot, entry_q_start, entry_q_len, items, num_items, mode,
                          scratch_s, scratch_a, H, D, V, 0, 0, 0, nullptr, nullptr, 0, 2,
                          static_cast<long long>(D) * V, static_cast<long long>(H) * D * V, stream);
}

// The recurrence for entries that bring ONE token (decode steps): the state is streamed, not held: thread
// (row group, column) walks its rows of the column once, eight loads in flight, S <- alpha S + k v written
// back as it goes, its share of o left in shared memory; then a warp per 32 columns adds the shares and
// applies norm, weight, gate and scale.  Few registers, so several blocks share an SM and the state's
// bytes bound the kernel, as keys and values bound decode attention.  Entry i is row q_start[i].
// What the step kernel can make itself instead of reading it: a rotation of q and k (retention), and the
// gates of a matrix memory with exponential gating (its decay, input scale and floor).
struct StepExtras {
    const float* rot_inv_freq;        // float32 [rot_dims / 2] or null: rotate pairs (i, i + rot_dims/2) of q and k
    int rot_dims;                     // by the angle float(position) * inv_freq[i]
    const int32_t* positions;
    float gate_cap;                   // > 0: a = exp(f + m - m'), e = exp(i - m'), floor = exp(-m') from the raw gates
    int i_off, f_off;                 // columns of the projection that hold them, one per head
    const float* i_bias;
    const float* f_bias;
    long long m_off;                  // where the running maximum m sits inside a head's state
};

// The log gates of a matrix memory: i = cap * tanh(z_i / cap), f = logsigmoid(cap * tanh(z_f / cap)).
__device__ __forceinline__ void recur_log_gates(float zi, float zf, float cap, float& ig, float& fg) {
    ig = cap * tanhf(zi / cap);
    const float c = cap * tanhf(zf / cap);
    fg = c < 0.0f ? c - log1pf(expf(c)) : -log1pf(expf(-c));
}

template <typename TO>
__global__ void gla_step_kernel(
    const float* __restrict__ proj, long long stride, int q_off, int k_off, int v_off, int g_off,
    const float* __restrict__ la, const float* __restrict__ norm_w, float eps, float q_scale, float out_scale,
    TO* __restrict__ out, long long out_stride, int out_off, float* __restrict__ state,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start, int H, int D, int V, int DG,
    int a_off, int rank, const float* __restrict__ w2t, const float* __restrict__ b2, float inv_tau,
    long long a_tok, long long a_head, long long a_chan, int normaliser, const RecurOpts opt, const StepExtras ex) {
    pdl_begin();
    extern __shared__ __align__(16) float smem[];
    const int VC = V + (normaliser ? 1 : 0);
    float* sq = smem;                 // [D]
    float* sk = sq + D;
    float* sa = sk + D;
    float* sv = sa + D;               // [V]
    float* part = sv + V;             // [DG][VC]
    float* red = part + DG * VC;      // 33, then 3 scalars of the gates
    float* a1 = red + 36;             // [rank]: the decay projection's first half, when the decays are made here
    const int entry = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const size_t row = static_cast<size_t>(entry_q_start[entry]);
    const float* pr = proj + row * stride;
    float* head_state = state + static_cast<size_t>(entry_slot[entry]) * opt.state_slot_stride + h * opt.state_head_stride;
    if (!la && rank > 0) {
        for (int j = tid; j < rank; j += blockDim.x) a1[j] = pr[a_off + j];
        __syncthreads();
    }
    if (ex.gate_cap > 0.0f && tid == 0) {
        float ig, fg;
        recur_log_gates(pr[ex.i_off + h] + ex.i_bias[h], pr[ex.f_off + h] + ex.f_bias[h], ex.gate_cap, ig, fg);
        const float m_old = head_state[ex.m_off];
        const float m_new = fmaxf(fg + m_old, ig);
        red[33] = expf(fg + m_old - m_new);
        red[34] = expf(ig - m_new);
        red[35] = expf(-m_new);
        head_state[ex.m_off] = m_new;
    }
    for (int d = tid; d < D; d += blockDim.x) {
        sq[d] = pr[q_off + h * D + d];
        sk[d] = pr[k_off + h * D + d];
        if (la) {
            sa[d] = la[row * a_tok + h * a_head + d * a_chan];       // the decay itself
        } else if (rank > 0) {                         // alpha = sigmoid(w2[c, :] . a1 + b2[c]) ^ (1 / tau), as gla_decay_kernel
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
    if (ex.rot_inv_freq) {                             // pairs (i, i + half) of q and k turn by position * inv_freq[i]
        const int half = ex.rot_dims >> 1;
        const float p = static_cast<float>(ex.positions[row]);
        for (int i = tid; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf(p * ex.rot_inv_freq[i], &sn, &cs);
            const float qu = sq[i], qv = sq[i + half], ku = sk[i], kv = sk[i + half];
            sq[i] = qu * cs - qv * sn;
            sq[i + half] = qv * cs + qu * sn;
            sk[i] = ku * cs - kv * sn;
            sk[i + half] = kv * cs + ku * sn;
        }
    }
    float floor_t = 0.0f;
    if (ex.gate_cap > 0.0f) {
        const float keep = red[33], put = red[34];
        floor_t = red[35];
        __syncthreads();                               // the rotation (if any) and red[] are settled
        for (int d = tid; d < D; d += blockDim.x) {
            sa[d] = keep;
            sk[d] *= put;
        }
    }
    __syncthreads();
    const bool active = tid < VC * DG;
    const int c = active ? tid % VC : 0, dg = active ? tid / VC : 0;
    const int rows = (D + DG - 1) / DG, d0 = dg * rows, d1 = min(D, d0 + rows);
    // column c < V of S has stride V; the normaliser column is contiguous after S
    float* S = c < V ? head_state + c : head_state + static_cast<size_t>(D) * V;
    const size_t ss = c < V ? V : 1;
    if (active) {
        const float vt = c < V ? sv[c] : 1.0f;
        float p = 0.0f;
        int d = d0;
        for (; d + 8 <= d1; d += 8) {
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = S[static_cast<size_t>(d + u) * ss];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                x[u] = sa[d + u] * x[u] + sk[d + u] * vt;
                S[static_cast<size_t>(d + u) * ss] = x[u];
                p += x[u] * sq[d + u];
            }
        }
        for (; d < d1; ++d) {
            const float x = sa[d] * S[static_cast<size_t>(d) * ss] + sk[d] * vt;
            S[static_cast<size_t>(d) * ss] = x;
            p += x * sq[d];
        }
        part[dg * VC + c] = p;
    }
    __syncthreads();
    float mul = q_scale;                               // q = W_q x * q_scale, applied to the finished sums
    if (normaliser) {
        float nq = part[V];
        for (int g2 = 1; g2 < DG; ++g2) nq += part[g2 * VC + V];
        mul = q_scale / (fmaxf(fabsf(nq * q_scale), floor_t) + 1e-6f);
    }
    __syncthreads();
    float sq2 = 0.0f;
    for (int i = tid; i < V; i += blockDim.x) {
        float o = part[i];
        for (int g2 = 1; g2 < DG; ++g2) o += part[g2 * VC + i];
        o *= mul;
        part[i] = o;
        sq2 += o * o;
    }
    const float total = block_sum(sq2, red);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(V) + eps);
    TO* orow = out + row * out_stride + out_off + h * V;
    const float* nw = norm_w ? norm_w + h * opt.norm_stride : nullptr;
    for (int i = tid; i < V; i += blockDim.x)
        orow[i] = from_f32<TO>(part[i] * inv * (nw ? nw[i] : 1.0f) * recur_gate(pr[g_off + h * V + i], opt.gate_kind) * out_scale);
}

// The general entry point of the step kernel.  `la` with strides (a_tok, a_head, a_chan): the decays as they
// are (a constant per head: 0, 1, 0).  la null and rank > 0: the low-rank decay projection is applied here.
// gate_cap > 0: the gates of a matrix memory are made here (a normaliser column is then kept, and m at m_off).
extern "C" int llm_recur_step(
    const float* proj, long long stride, int q_off, int k_off, int v_off, int g_off, const float* la,
    const float* norm_w, float eps, float q_scale, float out_scale, void* out, int out_dtype, long long out_stride,
    int out_off, float* state, const int32_t* entry_slot, const int32_t* entry_q_start, int num_entries, int H, int D,
    int V, int a_off, int rank, const float* w2t, const float* b2, float tau, long long a_tok, long long a_head,
    long long a_chan, int norm_stride, int gate_kind, long long state_head_stride, long long state_slot_stride,
    const float* rot_inv_freq, int rot_dims, const int32_t* positions, float gate_cap, int i_off, int f_off,
    const float* i_bias, const float* f_bias, uintptr_t stream) {
    if (num_entries <= 0) return LLM_OK;
    if (H <= 0 || D <= 0 || V <= 0 || H > 65535 || V > 1023) return LLM_REFUSED_SIZE;
    const int normaliser = gate_cap > 0.0f ? 1 : 0;
    if (!la && !normaliser && (!w2t || rank <= 0 || rank > 4096 || !(tau > 0.0f))) return LLM_REFUSED_SIZE;
    if (la || normaliser) rank = 0;
    if (normaliser && (!i_bias || !f_bias)) return LLM_REFUSED_SIZE;
    if (rot_inv_freq && (rot_dims <= 0 || rot_dims % 2 || rot_dims > D || !positions)) return LLM_REFUSED_SIZE;
    if (gate_kind < 0 || gate_kind > 2) return LLM_REFUSED_SIZE;
    const int VC = V + normaliser;
    if (state_head_stride < static_cast<long long>(D) * VC + normaliser) return LLM_REFUSED_SIZE;
    int DG = 256 / VC;
    if (DG < 1) DG = 1;
    if (DG > D) DG = D;
    const int threads = (VC * DG + 31) / 32 * 32;
    const size_t smem = (3 * static_cast<size_t>(D) + V + static_cast<size_t>(DG) * VC + 36 + rank) * sizeof(float);
    if (smem > 48 * 1024) return LLM_REFUSED_SIZE;
    const float inv_tau = rank > 0 ? 1.0f / tau : 0.0f;
    const RecurOpts opt = {0, 0, nullptr, nullptr, norm_stride, gate_kind, state_head_stride, state_slot_stride};
    const StepExtras ex = {rot_inv_freq, rot_dims, positions, gate_cap, i_off, f_off, i_bias, f_bias,
                           static_cast<long long>(D) * V + D};
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(num_entries, H);
    if (out_dtype == LLM_DT_F32)
        launch_pdl((gla_step_kernel<float>), grid, dim3(threads), smem, s, proj, stride, q_off, k_off, v_off, g_off, la, norm_w,
                   eps, q_scale, out_scale, static_cast<float*>(out), out_stride, out_off, state, entry_slot, entry_q_start,
                   H, D, V, DG, a_off, rank, w2t, b2, inv_tau, a_tok, a_head, a_chan, normaliser, opt, ex);
    else if (out_dtype == LLM_DT_BF16)
        launch_pdl((gla_step_kernel<bf16>), grid, dim3(threads), smem, s, proj, stride, q_off, k_off, v_off, g_off, la, norm_w,
                   eps, q_scale, out_scale, static_cast<bf16*>(out), out_stride, out_off, state, entry_slot, entry_q_start,
                   H, D, V, DG, a_off, rank, w2t, b2, inv_tau, a_tok, a_head, a_chan, normaliser, opt, ex);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

extern "C" int llm_gla_step(
    const float* proj, long long stride, int q_off, int k_off, int v_off, int g_off, const float* la,
    const float* norm_w, float eps, float q_scale, float out_scale, void* out, int out_dtype, long long out_stride,
    int out_off, float* state, const int32_t* entry_slot, const int32_t* entry_q_start, int num_entries, int H, int D,
    int V, int a_off, int rank, const float* w2t, const float* b2, float tau, uintptr_t stream) {
    // la null: the decays are computed here from the projection's columns a_off .. a_off + rank (w2t, b2, tau as
    // for llm_gla_decay), which saves a decode step one launch a layer
    if (!la && (!w2t || rank <= 0)) return LLM_REFUSED_SIZE;
    return llm_recur_step(proj, stride, q_off, k_off, v_off, g_off, la, norm_w, eps, q_scale, out_scale, out, out_dtype,
                          out_stride, out_off, state, entry_slot, entry_q_start, num_entries, H, D, V, a_off, rank, w2t,
                          b2, tau, static_cast<long long>(H) * D, D, 1, 0, 2, static_cast<long long>(D) * V,
                          static_cast<long long>(H) * D * V, nullptr, 0, nullptr, 0.0f, 0, 0, nullptr, nullptr, stream);
}

// chains: int32 [n, 3] = (entry, first scratch index, number of chunks); chunk c of the entry is scratch
// index first + c.  grid (n, H, blocks over D*V).
__global__ void gla_chain_kernel(float* __restrict__ state, float* __restrict__ scratch_s,
                                 const float* __restrict__ scratch_a, const int32_t* __restrict__ chains,
                                 const int32_t* __restrict__ entry_slot, int H, int D, int V, int VC,
                                 long long state_head_stride, long long state_slot_stride) {
    pdl_begin();
    const int entry = chains[3 * blockIdx.x];
    if (entry < 0) return;
    const int first = chains[3 * blockIdx.x + 1], n = chains[3 * blockIdx.x + 2];
    const int h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= D * VC) return;
    const int d = e < D * V ? e / V : e - D * V;         // S [D, V], then the normaliser n [D] when VC = V + 1
    const size_t per = static_cast<size_t>(D) * VC;
    float* st = state + static_cast<size_t>(entry_slot[entry]) * state_slot_stride + h * state_head_stride + e;
    float S = *st;
    for (int c0 = 0; c0 < n; c0 += 8) {              // eight chunks' loads in flight, then the chain through them
        float L[8], A[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const size_t at = static_cast<size_t>(first + min(c0 + i, n - 1)) * H + h;
            L[i] = scratch_s[at * per + e];
            A[i] = scratch_a[at * D + d];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c0 + i < n) {
                scratch_s[(static_cast<size_t>(first + c0 + i) * H + h) * per + e] = S;
                S = A[i] * S + L[i];
            }
    }
    *st = S;
}

// `normaliser` 1: a head's state is S [D, V] followed by n [D], and both are chained.
extern "C" int llm_recur_chain(float* state, float* scratch_s, const float* scratch_a, const int32_t* chains,
                               int num_chains, const int32_t* entry_slot, int H, int D, int V, int normaliser,
                               long long state_head_stride, long long state_slot_stride, uintptr_t stream) {
    if (num_chains <= 0) return LLM_OK;
    if (H <= 0 || D <= 0 || V <= 0 || H > 65535) return LLM_REFUSED_SIZE;
    const int VC = V + (normaliser ? 1 : 0);
    const int threads = 256;
    const int bz = (D * VC + threads - 1) / threads;
    if (bz > 65535) return LLM_REFUSED_SIZE;
    launch_pdl(gla_chain_kernel, dim3(num_chains, H, bz), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream),
               state, scratch_s, scratch_a, chains, entry_slot, H, D, V, VC, state_head_stride, state_slot_stride);
    return launch_status();
}

extern "C" int llm_gla_chain(float* state, float* scratch_s, const float* scratch_a, const int32_t* chains,
                             int num_chains, const int32_t* entry_slot, int H, int D, int V, uintptr_t stream) {
    return llm_recur_chain(state, scratch_s, scratch_a, chains, num_chains, entry_slot, H, D, V, 0,
                           static_cast<long long>(D) * V, static_cast<long long>(H) * D * V, stream);
}

// ---- what a recurrence with gates or a rotation needs before the scan over a prompt portion ------------
// recur_gates_kernel: per (entry, head), over the entry's tokens in order, from the raw gate columns of the
// projection: i = cap * tanh((z_i + b_i) / cap), f = logsigmoid(cap * tanh((z_f + b_f) / cap)), the running
// maximum m' = max(f + m, i) (m from the head's state, written back at the end), and per token
//     keep = exp(f + m - m'),   put = exp(i - m'),   floor = exp(-m')
// into three float32 [T, H] arrays (`gates` [3, T, H]).  Tokens are taken 128 at a time: every thread makes
// one token's log gates, one thread walks the maxima (an add and a max a token), every thread makes its token's
// exponentials and stores.
#define RG_TOKENS 128
__global__ void recur_gates_kernel(const float* __restrict__ proj, long long stride, int i_off, int f_off,
                                   const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                                   float* __restrict__ gates, long long num_tokens, float* __restrict__ state,
                                   long long m_off, long long state_head_stride, long long state_slot_stride,
                                   const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ entry_q_start,
                                   const int32_t* __restrict__ entry_q_len, int H) {
    pdl_begin();
    __shared__ float ig[RG_TOKENS], fg[RG_TOKENS], fl[RG_TOKENS], mx[RG_TOKENS];
    __shared__ float carry;
    const int entry = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const long long row0 = entry_q_start[entry];
    const int count = entry_q_len[entry];
    float* mp = state + static_cast<size_t>(entry_slot[entry]) * state_slot_stride + h * state_head_stride + m_off;
    if (tid == 0) carry = *mp;
    const float bi = i_bias[h], bf = f_bias[h];
    for (int done = 0; done < count; done += RG_TOKENS) {
        const int nb = min(RG_TOKENS, count - done);
        __syncthreads();
        if (tid < nb) {
            const float* pr = proj + (row0 + done + tid) * stride;
            recur_log_gates(pr[i_off + h] + bi, pr[f_off + h] + bf, cap, ig[tid], fg[tid]);
        }
        __syncthreads();
        if (tid == 0) {                                    // the chain itself is an add and a max a token
            float m = carry;
            for (int t = 0; t < nb; ++t) {
                const float m_new = fmaxf(fg[t] + m, ig[t]);
                fl[t] = m;                                 // the maximum that entered the token
                mx[t] = m_new;
                m = m_new;
            }
            carry = m;
        }
        __syncthreads();
        if (tid < nb) {                                    // the exponentials, a token a thread
            const long long at = (row0 + done + tid) * H + h;
            const float m_old = fl[tid], m_new = mx[tid];
            gates[at] = expf(fg[tid] + m_old - m_new);                        // keep
            gates[num_tokens * H + at] = expf(ig[tid] - m_new);               // put
            gates[2 * num_tokens * H + at] = expf(-m_new);                    // floor
        }
    }
    __syncthreads();
    if (tid == 0) *mp = carry;
}

extern "C" int llm_recur_gates(const float* proj, long long stride, int i_off, int f_off, const float* i_bias,
                               const float* f_bias, float cap, float* gates, long long num_tokens, float* state,
                               long long m_off, long long state_head_stride, long long state_slot_stride,
                               const int32_t* entry_slot, const int32_t* entry_q_start, const int32_t* entry_q_len,
                               int num_entries, int H, uintptr_t stream) {
    if (num_entries <= 0 || num_tokens <= 0) return LLM_OK;
    if (H <= 0 || H > 65535 || !(cap > 0.0f) || !i_bias || !f_bias) return LLM_REFUSED_SIZE;
    launch_pdl(recur_gates_kernel, dim3(num_entries, H), dim3(RG_TOKENS), 0, reinterpret_cast<cudaStream_t>(stream),
               proj, stride, i_off, f_off, i_bias, f_bias, cap, gates, num_tokens, state, m_off, state_head_stride,
               state_slot_stride, entry_slot, entry_q_start, entry_q_len, H);
    return launch_status();
}

// rotate_qk_kernel: in place on the float32 projection, pairs (i, i + dims/2) of every head of q and of k turn by
// the angle float(position) * inv_freq[i]; entries from `dims` on pass unchanged.  One block a token.
__global__ void rotate_qk_kernel(float* __restrict__ proj, long long stride, int q_off, int k_off, int heads_q,
                                 int heads_k, int D, int dims, const float* __restrict__ inv_freq,
                                 const int32_t* __restrict__ positions) {
    pdl_begin();
    const long long t = blockIdx.x;
    const int half = dims >> 1;
    const float p = static_cast<float>(positions[t]);
    float* row = proj + t * stride;
    const int pairs = (heads_q + heads_k) * half;
    for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        float* x = head < heads_q ? row + q_off + head * D : row + k_off + (head - heads_q) * D;
        float sn, cs;
        sincosf(p * inv_freq[i], &sn, &cs);
        const float u = x[i], v = x[i + half];
        x[i] = u * cs - v * sn;
        x[i + half] = v * cs + u * sn;
    }
}

extern "C" int llm_rotate_qk(float* proj, long long stride, int q_off, int k_off, int heads_q, int heads_k, int D,
                             int dims, const float* inv_freq, const int32_t* positions, int num_tokens,
                             uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (D <= 0 || dims <= 0 || dims % 2 || dims > D || heads_q < 0 || heads_k < 0) return LLM_REFUSED_SIZE;
    launch_pdl(rotate_qk_kernel, dim3(num_tokens), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), proj, stride,
               q_off, k_off, heads_q, heads_k, D, dims, inv_freq, positions);
    return launch_status();
}

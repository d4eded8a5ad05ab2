// Gated linear attention with a decay per key channel, as a recurrence over a float32 state per sequence and head:
//
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        (S is [dim, vdim]; the decay scales the rows)
//     o_t = S_t^T q_t
//     alpha_t = sigmoid(z_t)^(1/tau),  z_t = A2 (A1 h_t) + b
//
// followed by what stands between the recurrence and the output projection: each head's o is divided by its root
// mean square over vdim, multiplied by a weight [vdim] (one for all heads) and by silu(g_t).
//
// Everything of the recurrence is float32: the rows q, k, v, g and A1 h come as the float32 result of one product
// [T, P]; z, log alpha = -softplus(-z) / tau, alpha, the state and the sums are float32.  The state of a slot
// exists twice, [slot][2][heads][dim][vdim]: a step that begins at position p reads copy (p & 1) and writes copy
// ((p + n) & 1) after its n tokens.  A step of one token therefore never writes what it reads, so a recorded step
// that holds a sequence twice computes the same bits in both rows.
//
// One kernel serves a prompt's tokens and a single token.  A block takes a (work item, head): the item is a sequence's
// new tokens, or a segment of them.  A warp owns a run of key channels, a lane VP value columns (v = lane + 32 j), and
// each thread keeps its 64 elements of the state in registers; tokens are taken eight at a time: their q, k, alpha
// and v are prepared in shared memory by the whole block, the eight steps then run without a barrier (one
// broadcast load of 16 bytes, a channel's q, k and alpha, for 2 VP multiply-adds), and the block finishes their
// outputs together.
//
// A long prompt alone would leave most of the device idle (one block per sequence and head, its tokens in order), so
// its tokens are cut into segments that run side by side, in three launches:
//   1. every segment from a zero state: its own contribution U = sum_j diag(prod_{s>j} alpha_s) k_j v_j^T and the
//      product D of its decays (as the exponential of the summed logarithms);
//   2. per sequence, head and state element, over the segments in order: the state at each segment's start,
//      S <- D S + U, and the sequence's new state into the cache;
//   3. every segment again from its start state, now with outputs.
// The sums are those of the plain recurrence in another order, all in float32.
#include "common.cuh"

#define GLA_TOKENS 8         // tokens prepared together (few, so that two blocks share an SM: one prepares while one multiplies)
#define GLA_STATE_REGS 64    // elements of the state that one thread keeps

enum { GLA_WHOLE = 0, GLA_LOCAL = 1, GLA_OUTPUT = 3 };

struct GlaParams {
    const float* proj;       // [T, P]: q | k | v | g | a1 at the offsets below
    const void* a2;          // [heads * dim, rank], WT
    const float* a2_bias;    // [heads * dim]
    const float* norm_w;     // [vdim]
    float* state;            // [slots, 2, heads, dim, vdim]
    const int* seq_slot;     // [B]
    const int* seq_start;    // [B] position of the sequence's first new token
    const int* cu_q_len;     // [B + 1] rows of the step before each sequence
    void* out;               // [T, heads * vdim], OutT
    const int* seg_seq;      // [items] null: item b is all new tokens of sequence b; else the segment's sequence,
    const int* seg_begin;    //   its first token among the sequence's new tokens
    const int* seg_end;      //   and one past its last
    float* seg_local;        // [items, heads, dim, vdim] GLA_LOCAL writes U here
    float* seg_decay;        // [items, heads, dim]       GLA_LOCAL writes D here
    const float* seg_first;  // [items, heads, dim, vdim] GLA_OUTPUT starts from here
    float inv_tau, q_scale, eps;
    int P, off_q, off_k, off_v, off_g, off_a;
    int heads, dim, vdim, rank;
    int mode;
    int vpad, dpad, parts, dchunk;   // a block is `parts` warps; a warp keeps dchunk channels; dpad = parts * dchunk
    float* raw_out;                  // null, or [T, heads * vdim]: the value columns are cut into slices over blocks (a state
                                     // too large for one block's registers); the blocks leave o as it is here and a
                                     // second kernel norms and gates it
    int a2_shared;                   // the head's rows of A2 fit into shared memory beside the rest
    int a2_stride;                   // floats from one of those rows to the next
};

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(sigmoid(z)) = -softplus(-z) = min(z, 0) - log1p(exp(-|z|))
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// LOCAL: launch 1 of a segmented prompt, which needs neither queries nor outputs.
// SLICED: the value columns are cut over blocks (blockIdx.z) and the outputs go to raw_out.
template <typename WT, typename OutT, int VP, bool LOCAL, bool SLICED>
__global__ void __launch_bounds__(512) gla_scan_kernel(GlaParams p) {
    constexpr int DC = GLA_STATE_REGS / VP;
    extern __shared__ __align__(16) float sm[];
    after_previous_kernel();
    const int item = blockIdx.x, h = blockIdx.y;
    const int dim = p.dim, vdim = p.vdim, rank = p.rank;
    const int vpad = p.vpad, dpad = p.dpad, parts = p.parts, dchunk = p.dchunk;
    const int nthreads = blockDim.x;
    float4* s_qka = reinterpret_cast<float4*>(sm);     // [GLA_TOKENS][dpad]: (q, k, alpha, log alpha) of a channel
    float* s_v = sm + 4 * GLA_TOKENS * dpad;           // [GLA_TOKENS][vpad]
    float* s_a1 = s_v + GLA_TOKENS * vpad;             // [GLA_TOKENS][rank]
    float* s_o = s_a1 + GLA_TOKENS * rank;             // [GLA_TOKENS][parts][vpad]
    float* s_logsum = s_o + GLA_TOKENS * parts * vpad; // [dpad]
    float* s_a2 = s_logsum + ((dpad + 3) & ~3);                   // [dim][a2_stride] if a2_shared: row d is read by thread d; the stride
                                                       // (rank + 1, or rank + 4 where rows are read 16 bytes at a time) keeps
                                                       // a warp's loads on all banks
    const int a2_stride = p.a2_stride;

    const int b = p.seg_seq ? p.seg_seq[item] : item;
    const int row0 = p.cu_q_len[b], n_all = p.cu_q_len[b + 1] - row0;
    const int t_begin = p.seg_seq ? p.seg_begin[item] : 0, t_end = p.seg_seq ? p.seg_end[item] : n_all;
    const int start = p.seq_start[b];
    const size_t slot = (size_t)p.seq_slot[b];
    const size_t head_state = (size_t)dim * vdim;
    const float* s_in = nullptr;
    if (p.mode == GLA_WHOLE) s_in = p.state + ((slot * 2 + (start & 1)) * p.heads + h) * head_state;
    else if (p.mode == GLA_OUTPUT) s_in = p.seg_first + ((size_t)item * p.heads + h) * head_state;

    const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
    const int d0 = part * dchunk;
    const int v0 = SLICED ? blockIdx.z * vpad : 0, vcount = SLICED ? min(vpad, vdim - v0) : vdim;   // this block's value columns
    float S[DC][VP];
#pragma unroll
    for (int i = 0; i < DC; ++i)
#pragma unroll
        for (int j = 0; j < VP; ++j) {
            const int d = d0 + i, v = lane + 32 * j;
            S[i][j] = (s_in && i < dchunk && d < dim && v < vcount) ? s_in[(size_t)d * vdim + v0 + v] : 0.f;
        }
    for (int i = threadIdx.x; i < dpad; i += nthreads) s_logsum[i] = 0.f;
    // the padding of the rows stays zero: q = k = alpha = 0 there keeps a padded element of the state at zero
    for (int i = threadIdx.x; i < GLA_TOKENS * dpad; i += nthreads) s_qka[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = threadIdx.x; i < GLA_TOKENS * vpad; i += nthreads) s_v[i] = 0.f;

    const WT* a2 = (const WT*)p.a2 + (size_t)h * dim * rank;
    const float* a2_bias = p.a2_bias + h * dim;
    if (p.a2_shared)
        for (int i = threadIdx.x; i < dim * rank; i += nthreads) {
            const int d = i / rank, r = i - d * rank;
            s_a2[d * a2_stride + r] = to_f32<WT>(a2[i]);
        }

    for (int t0 = t_begin; t0 < t_end; t0 += GLA_TOKENS) {
        const int count = min(GLA_TOKENS, t_end - t0);
        const float* rows = p.proj + (size_t)(row0 + t0) * p.P;
        __syncthreads();                               // the outputs of the tokens before are finished
        for (int i = threadIdx.x; i < count * rank; i += nthreads) {
            const int t = i / rank, r = i - t * rank;
            s_a1[i] = rows[(size_t)t * p.P + p.off_a + r];
        }
        for (int i = threadIdx.x; i < count * vcount; i += nthreads) {
            const int t = i / vcount, c = i - t * vcount;
            s_v[t * vpad + c] = rows[(size_t)t * p.P + p.off_v + h * vdim + v0 + c];
        }
        __syncthreads();
        // four (token, channel) pairs a thread at a time: their loads go out together, then the arithmetic
        for (int base = 0; base < count * dim; base += 4 * nthreads) {
          float q4[4], k4[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = base + u * nthreads + threadIdx.x;
            const int t = i / dim, d = i - t * dim;
            const bool in = i < count * dim;
            q4[u] = (LOCAL || !in) ? 0.f : rows[(size_t)t * p.P + p.off_q + h * dim + d];
            k4[u] = in ? rows[(size_t)t * p.P + p.off_k + h * dim + d] : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = base + u * nthreads + threadIdx.x;
            if (i >= count * dim) break;
            const int t = i / dim, d = i - t * dim;
            const float qv = q4[u] * p.q_scale, kv = k4[u];
            float z = a2_bias[d];
            const float* a1 = s_a1 + t * rank;
            if (p.a2_shared && (rank & 3) == 0) {
                const float4* w = reinterpret_cast<const float4*>(s_a2 + d * a2_stride);
                const float4* x = reinterpret_cast<const float4*>(a1);
                for (int r = 0; r < rank / 4; ++r) {
                    const float4 wv = w[r], xv = x[r];
                    z += wv.x * xv.x;
                    z += wv.y * xv.y;
                    z += wv.z * xv.z;
                    z += wv.w * xv.w;
                }
            } else if (p.a2_shared) {
                const float* w = s_a2 + d * a2_stride;
                for (int r = 0; r < rank; ++r) z += w[r] * a1[r];
            } else {
                const WT* w = a2 + (size_t)d * rank;
                for (int r = 0; r < rank; ++r) z += to_f32<WT>(w[r]) * a1[r];
            }
            const float la = log_sigmoid(z) * p.inv_tau;
            s_qka[t * dpad + d] = make_float4(qv, kv, expf(la), la);
          }
        }
        __syncthreads();
        if (LOCAL)
            for (int d = threadIdx.x; d < dim; d += nthreads) {
                float sum = s_logsum[d];
                for (int t = 0; t < count; ++t) sum += s_qka[t * dpad + d].w;
                s_logsum[d] = sum;
            }
        for (int t = 0; t < count; ++t) {
            const float4* qka = s_qka + t * dpad + d0;
            float vt[VP], o[VP];
#pragma unroll
            for (int j = 0; j < VP; ++j) { vt[j] = s_v[t * vpad + lane + 32 * j]; o[j] = 0.f; }
#pragma unroll
            for (int i = 0; i < DC; ++i) {
                if (i < dchunk) {
                    const float4 c = qka[i];
#pragma unroll
                    for (int j = 0; j < VP; ++j) {
                        S[i][j] = c.z * S[i][j] + c.y * vt[j];
                        if (!LOCAL) o[j] += c.x * S[i][j];
                    }
                }
            }
            if (!LOCAL) {
#pragma unroll
                for (int j = 0; j < VP; ++j) s_o[(t * parts + part) * vpad + lane + 32 * j] = o[j];
            }
        }
        if (LOCAL) continue;
        __syncthreads();
        // a warp finishes a token: the parts of o added in order, the head's root mean square, weight and gate
        for (int t = part; t < count; t += parts) {
            if (SLICED) {
                float* raw = p.raw_out + ((size_t)(row0 + t0 + t) * p.heads + h) * vdim + v0;
                for (int c = lane; c < vcount; c += 32) {
                    float o = 0.f;
                    for (int s = 0; s < parts; ++s) o += s_o[(t * parts + s) * vpad + c];
                    raw[c] = o;
                }
                continue;
            }
            float ss = 0.f;
            for (int c = lane; c < vdim; c += 32) {
                float o = 0.f;
                for (int s = 0; s < parts; ++s) o += s_o[(t * parts + s) * vpad + c];
                s_o[(t * parts) * vpad + c] = o;
                ss += o * o;
            }
            ss = warp_sum(ss);
            const float rinv = 1.0f / sqrtf(ss / (float)vdim + p.eps);
            const float* g = rows + (size_t)t * p.P + p.off_g + h * vdim;
            OutT* out = (OutT*)p.out + ((size_t)(row0 + t0 + t) * p.heads + h) * vdim;
            for (int c = lane; c < vdim; c += 32) {
                const float gate = g[c];
                out[c] = from_f32<OutT>(s_o[(t * parts) * vpad + c] * rinv * p.norm_w[c] * (gate / (1.0f + expf(-gate))));
            }
        }
    }
    if (p.mode == GLA_OUTPUT) return;
    float* s_out = p.mode == GLA_WHOLE ? p.state + ((slot * 2 + ((start + n_all) & 1)) * p.heads + h) * head_state
                                       : p.seg_local + ((size_t)item * p.heads + h) * head_state;
#pragma unroll
    for (int i = 0; i < DC; ++i)
#pragma unroll
        for (int j = 0; j < VP; ++j) {
            const int d = d0 + i, v = lane + 32 * j;
            if (i < dchunk && d < dim && v < vcount) s_out[(size_t)d * vdim + v0 + v] = S[i][j];
        }
    if (LOCAL) {
        __syncthreads();
        for (int d = threadIdx.x; d < dim; d += nthreads) p.seg_decay[((size_t)item * p.heads + h) * dim + d] = expf(s_logsum[d]);
    }
}

// For a state cut into slices of value columns: out = raw / rms(raw over the head) * weight * silu(gate).
// grid (token, head), one warp.
template <typename OutT>
__global__ void gla_finish_kernel(const float* __restrict__ raw, const float* __restrict__ proj, const float* __restrict__ norm_w,
                                  OutT* __restrict__ out, int P, int off_g, int heads, int vdim, float eps) {
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const float* o = raw + ((size_t)t * heads + h) * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss += o[c] * o[c];
    ss = warp_sum(ss);
    const float rinv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const float* g = proj + (size_t)t * P + off_g + h * vdim;
    for (int c = lane; c < vdim; c += 32) {
        const float gate = g[c];
        out[((size_t)t * heads + h) * vdim + c] = from_f32<OutT>(o[c] * rinv * norm_w[c] * (gate / (1.0f + expf(-gate))));
    }
}

// How the value columns of a head's state are cut over blocks: columns per lane (1, 2, 4, 8) and slices of 32 times
// that many columns.  One slice wherever a block's registers hold the state (dim x vdim up to 32,768 with padding).
static inline bool gla_shape(int dim, int vdim, int* vp_out, int* slices_out) {
    int vp = (vdim + 31) / 32;
    vp = vp <= 1 ? 1 : vp == 2 ? 2 : vp <= 4 ? 4 : 8;
    while (vp > 1 && (dim + GLA_STATE_REGS / vp - 1) / (GLA_STATE_REGS / vp) > 16) vp /= 2;
    if ((dim + GLA_STATE_REGS / vp - 1) / (GLA_STATE_REGS / vp) > 16) return false;
    *vp_out = vp;
    *slices_out = (vdim + 32 * vp - 1) / (32 * vp);
    return true;
}

// The number of slices (1: no raw buffer is needed), or 0 for sizes that no launch takes.
FRB_API int frb_gla_value_slices(int dim, int vdim) {
    int vp = 0, slices = 0;
    return dim >= 1 && vdim >= 1 && gla_shape(dim, vdim, &vp, &slices) ? slices : 0;
}

// Launch 2 of a segmented prompt.  grid (sequence, head, tiles of 256 state elements).
__global__ void gla_combine_kernel(const float* __restrict__ seg_local, const float* __restrict__ seg_decay,
                                   float* __restrict__ seg_first, float* state, const int* __restrict__ seq_slot,
                                   const int* __restrict__ seq_start, const int* __restrict__ cu_q_len,
                                   const int* __restrict__ seq_seg0, int heads, int dim, int vdim) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int elements = dim * vdim;
    if (e >= elements) return;
    const int d = e / vdim;
    const int first = seq_seg0[b], count = seq_seg0[b + 1] - first;
    const int start = seq_start[b], n = cu_q_len[b + 1] - cu_q_len[b];
    const size_t slot = (size_t)seq_slot[b];
    float S = state[((slot * 2 + (start & 1)) * heads + h) * elements + e];
#pragma unroll 4
    for (int s = first; s < first + count; ++s) {
        const size_t at = (size_t)s * heads + h;
        seg_first[at * elements + e] = S;
        S = seg_decay[at * dim + d] * S + seg_local[at * elements + e];
    }
    state[((slot * 2 + ((start + n) & 1)) * heads + h) * elements + e] = S;
}

// num_items = num_seqs and null tables: every sequence whole.  With tables: the three launches of a segmented prompt;
// seg_scratch holds 2 * num_items * heads * dim * vdim + num_items * heads * dim floats.
FRB_API int frb_gla_scan(const float* proj, int P, int off_q, int off_k, int off_v, int off_g, int off_a,
                         const void* a2, int weight_dtype, const float* a2_bias, const float* norm_w, float* state,
                         const int* seq_slot, const int* seq_start, const int* cu_q_len, void* out, int out_dtype,
                         int num_seqs, int heads, int dim, int vdim, int rank, float tau, float q_scale, float eps,
                         const int* seg_seq, const int* seg_begin, const int* seg_end, const int* seq_seg0, int num_items,
                         float* seg_scratch, float* raw_out, int num_tokens, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(weight_dtype == out_dtype, "gla: the decay's matrix and the outputs must have one type");
    FRB_CHECK_ARG(dim >= 1 && vdim >= 1 && rank >= 1 && heads >= 1 && heads <= 65535, "gla: %d heads of %d x %d, rank %d",
                  heads, dim, vdim, rank);
    FRB_CHECK_ARG(tau > 0.f, "gla: tau %f", (double)tau);
    int vp = 0, slices = 0;
    FRB_CHECK_ARG(gla_shape(dim, vdim, &vp, &slices), "gla: %d key channels a head are more than a block's registers hold (1,024)", dim);
    FRB_CHECK_ARG(slices == 1 || raw_out, "gla: a state of %d x %d per head is cut into %d slices and needs the raw buffer", dim, vdim, slices);
    FRB_CHECK_ARG(slices <= 65535, "gla: %d slices", slices);
    GlaParams p;
    p.proj = proj; p.a2 = a2; p.a2_bias = a2_bias; p.norm_w = norm_w; p.state = state; p.seq_slot = seq_slot;
    p.seq_start = seq_start; p.cu_q_len = cu_q_len; p.out = out; p.inv_tau = 1.0f / tau; p.q_scale = q_scale; p.eps = eps;
    p.P = P; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v; p.off_g = off_g; p.off_a = off_a;
    p.heads = heads; p.dim = dim; p.vdim = vdim; p.rank = rank;
    p.vpad = 32 * vp;                                     // value columns of a block
    p.raw_out = slices > 1 ? raw_out : nullptr;
    const int most = GLA_STATE_REGS / vp;                 // channels a warp can keep
    int parts = (dim + most - 1) / most;
    if (parts < 8) parts = dim < 8 ? dim : 8;             // eight warps where the sizes allow
    p.parts = parts;
    p.dchunk = (dim + parts - 1) / parts;
    p.dpad = p.parts * p.dchunk;
    size_t smem = ((size_t)GLA_TOKENS * (4 * p.dpad + p.vpad + rank) + (size_t)GLA_TOKENS * parts * p.vpad + ((p.dpad + 3) & ~3)) * sizeof(float);
    p.a2_stride = rank % 4 == 0 ? rank + 4 : rank + 1;
    const size_t a2_bytes = (size_t)dim * p.a2_stride * sizeof(float);
    p.a2_shared = smem + a2_bytes <= 200 * 1024;          // (the registers of the state leave an SM one block of 256 threads anyway)
    if (p.a2_shared) smem += a2_bytes;
    FRB_CHECK_ARG(smem <= 200 * 1024, "gla: %d x %d per head with rank %d needs more than 200 KB of shared memory", dim, vdim, rank);
    const bool segmented = seg_seq != nullptr;
    FRB_CHECK_ARG(!segmented || (seg_begin && seg_end && seq_seg0 && seg_scratch && num_items > 0), "gla: segment tables are incomplete");
    const size_t per_item = (size_t)heads * dim * vdim;
    p.seg_seq = seg_seq; p.seg_begin = seg_begin; p.seg_end = seg_end;
    p.seg_local = segmented ? seg_scratch : nullptr;
    float* seg_first = segmented ? seg_scratch + (size_t)num_items * per_item : nullptr;
    p.seg_first = seg_first;
    p.seg_decay = segmented ? seg_scratch + 2 * (size_t)num_items * per_item : nullptr;
    const dim3 grid(segmented ? num_items : num_seqs, heads, slices), block(32 * parts);
#define FRB_GLA_LAUNCH(VP)                                                                                            \
    do {                                                                                                              \
        auto kernel = slices > 1 ? gla_scan_kernel<WT, OutT, VP, false, true> : gla_scan_kernel<WT, OutT, VP, false, false>; \
        auto local = slices > 1 ? gla_scan_kernel<WT, OutT, VP, true, true> : gla_scan_kernel<WT, OutT, VP, true, false>;   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(local, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        if (!segmented) {                                                                                             \
            p.mode = GLA_WHOLE;                                                                                       \
            launch_dependent(kernel, grid, block, smem, stream, p);                                                   \
        } else {                                                                                                      \
            p.mode = GLA_LOCAL;                                                                                       \
            local<<<grid, block, smem, stream>>>(p);                                                                  \
            gla_combine_kernel<<<dim3(num_seqs, heads, (dim * vdim + 255) / 256), 256, 0, stream>>>(                  \
                p.seg_local, p.seg_decay, seg_first, state, seq_slot, seq_start, cu_q_len, seq_seg0, heads, dim, vdim); \
            p.mode = GLA_OUTPUT;                                                                                      \
            kernel<<<grid, block, smem, stream>>>(p);                                                                 \
        }                                                                                                             \
        if (p.raw_out)                                                                                                \
            gla_finish_kernel<OutT><<<dim3(num_tokens, heads), 32, 0, stream>>>(p.raw_out, proj, norm_w, (OutT*)out, P, \
                                                                               off_g, heads, vdim, eps);             \
    } while (0)
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        typedef OutT WT;                                  // the decay's matrix is held in the type of the outputs
        if (vp == 1) FRB_GLA_LAUNCH(1); else if (vp == 2) FRB_GLA_LAUNCH(2); else if (vp == 4) FRB_GLA_LAUNCH(4); else FRB_GLA_LAUNCH(8);
    });
#undef FRB_GLA_LAUNCH
    FRB_RETURN_LAUNCH("gla_scan");
}

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
// This file has the scan that serves any sizes: one block per (sequence, head) walks the sequence's new tokens in
// order, a prompt's or a single one.  A thread owns a value column v and a run of key channels and keeps its part of
// the state in registers; tokens are taken sixteen at a time: their q, k, alpha and v are prepared in shared memory by
// the whole block, the sixteen steps then run without a barrier, and the block finishes their outputs together.
#include "common.cuh"

#define GLA_TOKENS 16        // tokens prepared together
#define GLA_CHANNELS 64      // most key channels of the state that one thread keeps

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
    float inv_tau, q_scale, eps;
    int P, off_q, off_k, off_v, off_g, off_a;
    int heads, dim, vdim, rank;
    int vpad, dsplit, dchunk;   // threads are [dsplit][vpad]; a thread keeps dchunk channels
};

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(sigmoid(z)) = -softplus(-z) = min(z, 0) - log1p(exp(-|z|))
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

template <typename WT, typename OutT>
__global__ void gla_scan_kernel(GlaParams p) {
    extern __shared__ float sm[];
    after_previous_kernel();
    const int b = blockIdx.x, h = blockIdx.y;
    const int dim = p.dim, vdim = p.vdim, rank = p.rank;
    const int vpad = p.vpad, dsplit = p.dsplit, dchunk = p.dchunk;
    const int nthreads = blockDim.x;
    float* s_q = sm;                                   // [GLA_TOKENS][dim]
    float* s_k = s_q + GLA_TOKENS * dim;
    float* s_a = s_k + GLA_TOKENS * dim;
    float* s_v = s_a + GLA_TOKENS * dim;               // [GLA_TOKENS][vdim]
    float* s_a1 = s_v + GLA_TOKENS * vdim;             // [GLA_TOKENS][rank]
    float* s_o = s_a1 + GLA_TOKENS * rank;             // [GLA_TOKENS][dsplit][vpad]

    const int row0 = p.cu_q_len[b], n = p.cu_q_len[b + 1] - row0;
    const int start = p.seq_start[b];
    const size_t slot = (size_t)p.seq_slot[b];
    const size_t head_state = (size_t)dim * vdim;
    const float* s_in = p.state + ((slot * 2 + (start & 1)) * p.heads + h) * head_state;
    float* s_out = p.state + ((slot * 2 + ((start + n) & 1)) * p.heads + h) * head_state;

    const int v = threadIdx.x % vpad, part = threadIdx.x / vpad;
    const int d0 = part * dchunk;
    const bool owner = v < vdim && part < dsplit;
    float S[GLA_CHANNELS];
#pragma unroll
    for (int i = 0; i < GLA_CHANNELS; ++i)
        S[i] = (owner && i < dchunk && d0 + i < dim) ? s_in[(size_t)(d0 + i) * vdim + v] : 0.f;

    const WT* a2 = (const WT*)p.a2 + (size_t)h * dim * rank;
    const float* a2_bias = p.a2_bias + h * dim;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = nthreads >> 5;

    for (int t0 = 0; t0 < n; t0 += GLA_TOKENS) {
        const int count = min(GLA_TOKENS, n - t0);
        const float* rows = p.proj + (size_t)(row0 + t0) * p.P;
        __syncthreads();                               // the outputs of the tokens before are finished
        for (int i = threadIdx.x; i < count * rank; i += nthreads) {
            const int t = i / rank, r = i - t * rank;
            s_a1[i] = rows[(size_t)t * p.P + p.off_a + r];
        }
        for (int i = threadIdx.x; i < count * vdim; i += nthreads) {
            const int t = i / vdim, c = i - t * vdim;
            s_v[i] = rows[(size_t)t * p.P + p.off_v + h * vdim + c];
        }
        for (int i = threadIdx.x; i < count * dim; i += nthreads) {
            const int t = i / dim, d = i - t * dim;
            s_q[i] = rows[(size_t)t * p.P + p.off_q + h * dim + d] * p.q_scale;
            s_k[i] = rows[(size_t)t * p.P + p.off_k + h * dim + d];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < count * dim; i += nthreads) {
            const int t = i / dim, d = i - t * dim;
            float z = a2_bias[d];
            const WT* w = a2 + (size_t)d * rank;
            const float* a1 = s_a1 + t * rank;
            for (int r = 0; r < rank; ++r) z += to_f32<WT>(w[r]) * a1[r];
            s_a[i] = expf(log_sigmoid(z) * p.inv_tau);
        }
        __syncthreads();
        if (owner) {
            for (int t = 0; t < count; ++t) {
                const float* q = s_q + t * dim + d0;
                const float* k = s_k + t * dim + d0;
                const float* a = s_a + t * dim + d0;
                const float vt = s_v[t * vdim + v];
                float o = 0.f;
#pragma unroll
                for (int i = 0; i < GLA_CHANNELS; ++i) {
                    if (i < dchunk && d0 + i < dim) {
                        S[i] = a[i] * S[i] + k[i] * vt;
                        o += q[i] * S[i];
                    }
                }
                s_o[(t * dsplit + part) * vpad + v] = o;
            }
        }
        __syncthreads();
        // a warp finishes a token: the parts of o added in order, the head's root mean square, weight and gate
        for (int t = warp; t < count; t += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < vdim; c += 32) {
                float o = 0.f;
                for (int s = 0; s < dsplit; ++s) o += s_o[(t * dsplit + s) * vpad + c];
                s_o[(t * dsplit) * vpad + c] = o;
                ss += o * o;
            }
            ss = warp_sum(ss);
            const float rinv = 1.0f / sqrtf(ss / (float)vdim + p.eps);
            const float* g = rows + (size_t)t * p.P + p.off_g + h * vdim;
            OutT* out = (OutT*)p.out + ((size_t)(row0 + t0 + t) * p.heads + h) * vdim;
            for (int c = lane; c < vdim; c += 32) {
                const float gate = g[c];
                out[c] = from_f32<OutT>(s_o[(t * dsplit) * vpad + c] * rinv * p.norm_w[c] * (gate / (1.0f + expf(-gate))));
            }
        }
    }
    if (owner) {
#pragma unroll
        for (int i = 0; i < GLA_CHANNELS; ++i)
            if (i < dchunk && d0 + i < dim) s_out[(size_t)(d0 + i) * vdim + v] = S[i];
    }
}

FRB_API int frb_gla_scan(const float* proj, int P, int off_q, int off_k, int off_v, int off_g, int off_a,
                         const void* a2, int weight_dtype, const float* a2_bias, const float* norm_w, float* state,
                         const int* seq_slot, const int* seq_start, const int* cu_q_len, void* out, int out_dtype,
                         int num_seqs, int heads, int dim, int vdim, int rank, float tau, float q_scale, float eps,
                         cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(dim >= 1 && vdim >= 1 && rank >= 1 && heads >= 1 && heads <= 65535, "gla: %d heads of %d x %d, rank %d",
                  heads, dim, vdim, rank);
    FRB_CHECK_ARG(tau > 0.f, "gla: tau %f", (double)tau);
    GlaParams p;
    p.proj = proj; p.a2 = a2; p.a2_bias = a2_bias; p.norm_w = norm_w; p.state = state; p.seq_slot = seq_slot;
    p.seq_start = seq_start; p.cu_q_len = cu_q_len; p.out = out; p.inv_tau = 1.0f / tau; p.q_scale = q_scale; p.eps = eps;
    p.P = P; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v; p.off_g = off_g; p.off_a = off_a;
    p.heads = heads; p.dim = dim; p.vdim = vdim; p.rank = rank;
    p.vpad = (vdim + 31) / 32 * 32;
    FRB_CHECK_ARG(p.vpad <= 1024, "gla: a value head of %d", vdim);
    int dsplit = (dim + GLA_CHANNELS - 1) / GLA_CHANNELS;
    const int want = 256 / p.vpad;                       // about 256 threads where the sizes allow
    if (dsplit < want) dsplit = want < dim ? want : dim;
    FRB_CHECK_ARG(dsplit * p.vpad <= 1024, "gla: a state of %d x %d per head needs more than 1024 threads", dim, vdim);
    p.dsplit = dsplit;
    p.dchunk = (dim + dsplit - 1) / dsplit;
    const size_t smem = ((size_t)GLA_TOKENS * (3 * dim + vdim + rank) + (size_t)GLA_TOKENS * dsplit * p.vpad) * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "gla: %d x %d per head with rank %d needs more than 200 KB of shared memory", dim, vdim, rank);
    FRB_DISPATCH_DTYPE(weight_dtype, WT, FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        auto kernel = gla_scan_kernel<WT, OutT>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dependent(kernel, dim3(num_seqs, heads), dim3(dsplit * p.vpad), smem, stream, p);
    }));
    FRB_RETURN_LAUNCH("gla_scan");
}

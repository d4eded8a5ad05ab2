// Recurrences over a float32 state per sequence, and the short causal convolution that stands in front of them.
//
//   causal_conv      out[t, c] = act(bias[c] + sum_k taps[c, k] * in[t - (K-1) + k, c]), the inputs before a step's first
//                    token coming from the state (the last K-1 inputs of the sequence; zeros for a new sequence); two
//                    kernels: the rows that see only their own step, and each sequence's first rows with the state
//   selective_scan   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  y silu(z)
//   gated_recurrence a = exp(-g r softplus(lam)),  S <- a S + sqrt(1 - a^2) i u,  out = S * act(y)    (per channel)
//   state_space_scan per head: S <- exp(-exp(A_log) dt) S + dt B x^T (S is [N, vdim]);  y = S^T C + D x;  y silu(z)
//   group_rms_norm   rows divided, in equal parts, by each part's root mean square, times a weight
//
// Everything here is float32: the rows come as the float32 results of the projections, the state lives in float32.
// The state of a slot exists twice, [slot][2][floats]: a step that begins at position p reads copy (p & 1) and writes
// copy ((p + n) & 1) after its n tokens, so a step of one token never writes what it reads and a recorded step that
// holds a sequence twice computes the same bits in both rows.  A prompt's step may read and write the same copy: every
// element of the state is then read and written by one thread only, which reads before it writes.
//
// A decay a = exp(l) with l close to 0 is kept as a - 1 = expm1(l) and applied as S + (a - 1) S: rounded to float32, a
// itself would lose its distance from 1, by the same amount at every step, and over a thousand tokens that bias adds
// up to 1e-4 of the state; the rounding of S + (a - 1) S has no preferred direction.
#include "common.cuh"

#define SCAN_TOKENS 8        // tokens whose rows are asked for together

struct SeqTables {
    const int* seq_slot;     // [B]
    const int* seq_start;    // [B] position of the sequence's first new token
    const int* cu_q_len;     // [B + 1] rows of the step before each sequence
};

struct StatePlace {
    float* base;             // [slots][2][copy_floats]
    long long copy_floats;   // floats of one copy of a slot's state
    long long offset;        // where, within a copy, this kernel's part begins
};

__device__ __forceinline__ float* state_at(const StatePlace& s, int slot, int copy) {
    return s.base + ((size_t)slot * 2 + copy) * s.copy_floats + s.offset;
}

__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
// silu for a result that is rounded to bfloat16 right away: the fast exponential and division (errors of 1e-6)
template <typename OutT> __device__ __forceinline__ float silu_for(float v) { return silu_f(v); }
template <> __device__ __forceinline__ float silu_for<bf16>(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
// exp(x) - 1 for x <= 0 (a decay less one): four terms of the series where the result is small (the fifth is below
// 1e-8 of it under 1/32), else the fast exponential, whose error of a few 1e-7 of the decay then matters as little as
// the rounding of the state itself.
__device__ __forceinline__ float decay_less_one(float x) {
    const float series = x * fmaf(x, fmaf(x, fmaf(x, 1.0f / 24.0f, 1.0f / 6.0f), 0.5f), 1.0f);
    return x > -0.03125f ? series : __expf(x) - 1.0f;
}

__device__ __forceinline__ float gelu_tanh_f(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

// ---------------------------------------------------------------------------------------------------- causal_conv

#define CONV_MAX_TAPS 16

struct ConvParams {
    const float* in;         // [T, in_stride]; channel c at column in_offset + c
    const float* in_bias;    // [C] or null: added to every input
    const float* taps;       // [C, K]; the last column weighs the current token
    const float* bias;       // [C] or null
    const int* tok_seq;      // [T]
    SeqTables seq;
    StatePlace state;        // [K - 1][C]: the last inputs, oldest first
    float* out32;            // [T, C]
    void* out_typed;         // null, or [T, C] in the model dtype
    int in_stride, in_offset, channels, taps_count, activation, num_rows;
    int rows_per_thread;     // CONV_ROWS for a step of many rows, 1 for a step of few (one token a sequence)
};

__device__ __forceinline__ float conv_activation(float v, int activation) { return activation == 1 ? silu_f(v) : v; }

#define CONV_ROWS 8          // rows of the step that one thread takes, one after the other, for its channel

// The rows that see only inputs of their own step (row i >= K-1 of its sequence).  A thread takes CONV_ROWS rows of the
// step for one channel: the inputs of all of them (the rows themselves and the K-1 before the first) are asked for
// before the first is used, and every row's window is a run of those registers.  Rows 0 .. K-2 of a sequence are the
// other kernel's.
template <typename OutT>
__global__ void __launch_bounds__(128) causal_conv_rows_kernel(ConvParams p) {
    after_previous_kernel();
    const int c = blockIdx.y * 128 + threadIdx.x;
    if (c >= p.channels) return;
    const int K = p.taps_count;
    const int r_begin = blockIdx.x * p.rows_per_thread, r_end = min(p.num_rows, r_begin + p.rows_per_thread);
    const float in_bias = p.in_bias ? p.in_bias[c] : 0.f;
    const float* in = p.in + p.in_offset + c;
    // vals[m]: the input of row r_begin - (MAX - 1) + m; a row's window is right aligned, the newest last
    float vals[CONV_ROWS + CONV_MAX_TAPS - 1];
#pragma unroll
    for (int m = 0; m < CONV_ROWS + CONV_MAX_TAPS - 1; ++m) {
        const int r = r_begin - (CONV_MAX_TAPS - 1) + m;
        vals[m] = (m >= CONV_MAX_TAPS - K && r >= 0 && r < r_end) ? in[(size_t)r * p.in_stride] + in_bias : 0.f;
    }
    float w[CONV_MAX_TAPS];                    // right aligned like the windows: w[MAX - K + k] is tap k
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = j >= CONV_MAX_TAPS - K ? p.taps[(size_t)c * K + j - (CONV_MAX_TAPS - K)] : 0.f;
    const float bias = p.bias ? p.bias[c] : 0.f;
    OutT* typed = (OutT*)p.out_typed;
    // most threads' rows lie in one sequence: its tables are then looked up once, not row by row
    const int b_first = p.tok_seq[r_begin], b_last = p.tok_seq[r_end - 1];
    const int row0_first = p.seq.cu_q_len[b_first];
    const bool one_sequence = b_first == b_last;
#pragma unroll
    for (int q = 0; q < CONV_ROWS; ++q) {
        const int r = r_begin + q;
        if (r < r_end) {
            const int row0 = one_sequence ? row0_first : p.seq.cu_q_len[p.tok_seq[r]];
            if (r - row0 >= K - 1) {
                float acc = bias;
#pragma unroll
                for (int j = 0; j < CONV_MAX_TAPS; ++j) acc = fmaf(w[j], vals[q + j], acc);
                acc = conv_activation(acc, p.activation);
                p.out32[(size_t)r * p.channels + c] = acc;
                if (typed) typed[(size_t)r * p.channels + c] = from_f32<OutT>(acc);
            }
        }
    }
}

// A thread per (sequence, channel) does all that touches the state: the outputs of the sequence's first K-1 new rows
// (the only ones that see inputs from before the step) and the new state.  It reads the old state before it writes.
template <typename OutT>
__global__ void __launch_bounds__(128) causal_conv_heads_kernel(ConvParams p) {
    after_previous_kernel();
    const int c = blockIdx.y * 128 + threadIdx.x;
    const int b = blockIdx.x;
    if (c >= p.channels) return;
    const int K = p.taps_count;
    const float bias = p.bias ? p.bias[c] : 0.f, in_bias = p.in_bias ? p.in_bias[c] : 0.f;
    const float* in = p.in + p.in_offset + c;
    OutT* typed = (OutT*)p.out_typed;
    const int row0 = p.seq.cu_q_len[b], n = p.seq.cu_q_len[b + 1] - row0;
    const int start = p.seq.seq_start[b], slot = p.seq.seq_slot[b];
    const float* old_tail = state_at(p.state, slot, start & 1);
    float* new_tail = state_at(p.state, slot, (start + n) & 1);
    // hist[m], m < K-1: the inputs before the step; hist[MAX + j]: the step's own input j, for the rows handled here
    float hist[2 * CONV_MAX_TAPS];
#pragma unroll
    for (int m = 0; m < CONV_MAX_TAPS; ++m) hist[m] = m < K - 1 ? old_tail[(size_t)m * p.channels + c] : 0.f;
    const int own = min(n, K - 1);
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j)
        hist[CONV_MAX_TAPS + j] = j < own ? in[(size_t)(row0 + j) * p.in_stride] + in_bias : 0.f;
    for (int j = 0; j < own; ++j) {
        float acc = bias;
        for (int k = 0; k < K; ++k) {
            const int at = j - (K - 1) + k;                       // index among the step's inputs; negative: before it
            const float v = at >= 0 ? hist[CONV_MAX_TAPS + at] : hist[K - 1 + at];
            acc = fmaf(p.taps[(size_t)c * K + k], v, acc);
        }
        acc = conv_activation(acc, p.activation);
        p.out32[(size_t)(row0 + j) * p.channels + c] = acc;
        if (typed) typed[(size_t)(row0 + j) * p.channels + c] = from_f32<OutT>(acc);
    }
    for (int m = 0; m < K - 1; ++m) {
        const int at = n - (K - 1) + m;                           // the step's input that becomes entry m of the new state
        float v;
        if (at < 0) v = hist[K - 1 + at];
        else if (at < own) v = hist[CONV_MAX_TAPS + at];
        else v = in[(size_t)(row0 + at) * p.in_stride] + in_bias;
        new_tail[(size_t)m * p.channels + c] = v;
    }
}

FRB_API int frb_causal_conv(const float* in, int in_stride, int in_offset, const float* in_bias, const float* taps,
                            const float* bias, const int* tok_seq, const int* seq_slot, const int* seq_start,
                            const int* cu_q_len, float* state, long long copy_floats, long long state_offset, float* out32,
                            void* out_typed, int typed_dtype, int num_rows, int num_seqs, int channels, int taps_count,
                            int activation, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(taps_count >= 1 && taps_count <= CONV_MAX_TAPS, "causal_conv: %d taps are outside 1..%d", taps_count,
                  CONV_MAX_TAPS);
    ConvParams p;
    p.in = in; p.in_bias = in_bias; p.taps = taps; p.bias = bias; p.tok_seq = tok_seq;
    p.seq = SeqTables{seq_slot, seq_start, cu_q_len};
    p.state = StatePlace{state, copy_floats, state_offset};
    p.out32 = out32; p.out_typed = out_typed; p.in_stride = in_stride; p.in_offset = in_offset; p.channels = channels;
    p.taps_count = taps_count; p.activation = activation; p.num_rows = num_rows;
    FRB_CHECK_ARG((channels + 127) / 128 <= 65535, "causal_conv: %d channels exceed the grid", channels);
    p.rows_per_thread = num_rows >= 2048 ? CONV_ROWS : 1;
    dim3 grid((num_rows + p.rows_per_thread - 1) / p.rows_per_thread, (channels + 127) / 128);
    dim3 heads(num_seqs, (channels + 127) / 128);
    FRB_DISPATCH_DTYPE(typed_dtype, OutT, {
        // one token a sequence: no row sees only its own step (unless there is one tap, and then no state)
        if (taps_count == 1 || num_rows > num_seqs) launch_dependent(causal_conv_rows_kernel<OutT>, grid, dim3(128), 0, stream, p);
        if (taps_count > 1) launch_dependent(causal_conv_heads_kernel<OutT>, heads, dim3(128), 0, stream, p);
    });
    FRB_RETURN_LAUNCH("causal_conv");
}

// ---------------------------------------------------------------------------------------------------- selective_scan

#define SEL_BLOCK 128

// x <- softplus(x + bias), row by row: the step sizes of the selective scan, made once for all the lanes that share them
__global__ void __launch_bounds__(256) softplus_bias_kernel(float* __restrict__ x, const float* __restrict__ bias, int num_rows,
                                                            int width) {
    after_previous_kernel();
    for (int row = blockIdx.x; row < num_rows; row += gridDim.x)
        for (int c = threadIdx.x; c < width; c += 256) {
            const size_t i = (size_t)row * width + c;
            x[i] = softplus_f(x[i] + bias[c]);
        }
}

FRB_API int frb_softplus_bias(float* x, const float* bias, int num_rows, int width, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    launch_dependent(softplus_bias_kernel, dim3(num_rows < 2368 ? num_rows : 2368), dim3(256), 0, stream, x, bias, num_rows, width);
    FRB_RETURN_LAUNCH("softplus_bias");
}

struct SelScanParams {
    const float* xz;         // [T, xz_stride]: z of channel c at z_offset + c
    const float* x;          // [T, inner]: the convolution's output
    const float* low;        // [T, low_stride]: B at b_offset, C at c_offset
    const float* dt;         // [T, inner]: the step size (after bias and softplus)
    const float* a_log;      // [inner, N]
    const float* d;          // [inner]
    SeqTables seq;
    StatePlace state;        // [inner][N]
    void* out;               // [T, inner]
    int xz_stride, z_offset, low_stride, b_offset, c_offset, inner, N, split;
};

// A channel's N state elements lie on `split` neighbouring lanes (a power of two), REGS each.  Few elements a lane
// (REGS 2 or 4) spread a prompt of few sequences over the whole device; many (16) spare the lanes' additions where a
// step has channels enough.
template <typename OutT, int REGS>
__global__ void __launch_bounds__(SEL_BLOCK) selective_scan_kernel(SelScanParams p) {
    extern __shared__ float sm[];
    after_previous_kernel();
    const int N = p.N, split = p.split;
    float* s_b = sm;                        // [SCAN_TOKENS][N]
    float* s_c = sm + SCAN_TOKENS * N;      // [SCAN_TOKENS][N]
    const int b = blockIdx.y;
    const int per_block = SEL_BLOCK / split;
    const int part = threadIdx.x % split;
    const int c = blockIdx.x * per_block + threadIdx.x / split;
    const bool live = c < p.inner;
    const int row0 = p.seq.cu_q_len[b], n_tok = p.seq.cu_q_len[b + 1] - row0;
    const int start = p.seq.seq_start[b], slot = p.seq.seq_slot[b];
    const int n0 = part * REGS;
    float S[REGS], A[REGS];
    const float* s_in = state_at(p.state, slot, start & 1);
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const bool has = live && n0 + i < N;
        S[i] = has ? s_in[(size_t)c * N + n0 + i] : 0.f;
        A[i] = has ? -expf(p.a_log[(size_t)c * N + n0 + i]) : 0.f;
    }
    const float dskip = live ? p.d[c] : 0.f;
    OutT* out = (OutT*)p.out;
    for (int t0 = 0; t0 < n_tok; t0 += SCAN_TOKENS) {
        const int count = min(SCAN_TOKENS, n_tok - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < count * N; i += SEL_BLOCK) {
            const int t = i / N, n = i - t * N;
            const float* row = p.low + (size_t)(row0 + t0 + t) * p.low_stride;
            s_b[i] = row[p.b_offset + n];
            s_c[i] = row[p.c_offset + n];
        }
        float dtv[SCAN_TOKENS], xv[SCAN_TOKENS], zv[SCAN_TOKENS];
#pragma unroll
        for (int t = 0; t < SCAN_TOKENS; ++t) {
            const bool has = live && t < count;
            const size_t row = (size_t)(row0 + t0 + t);
            dtv[t] = has ? p.dt[row * p.inner + c] : 0.f;
            xv[t] = has ? p.x[row * p.inner + c] : 0.f;
            zv[t] = has && part == 0 ? p.xz[row * p.xz_stride + p.z_offset + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < SCAN_TOKENS; ++t) {
            if (t < count) {
                const float step = dtv[t];
                const float sx = step * xv[t];
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < REGS; ++i) {
                    if (n0 + i < N) {
                        S[i] = fmaf(decay_less_one(step * A[i]), S[i], S[i]) + sx * s_b[t * N + n0 + i];
                        y = fmaf(S[i], s_c[t * N + n0 + i], y);
                    }
                }
                for (int o = 1; o < split; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (live && part == 0)
                    out[(size_t)(row0 + t0 + t) * p.inner + c] = from_f32<OutT>((y + dskip * xv[t]) * silu_for<OutT>(zv[t]));
            }
        }
    }
    if (live) {
        float* s_out = state_at(p.state, slot, (start + n_tok) & 1);
#pragma unroll
        for (int i = 0; i < REGS; ++i)
            if (n0 + i < N) s_out[(size_t)c * N + n0 + i] = S[i];
    }
}

static inline int split_for(int N, int regs) {
    int split = 1;
    while (split * regs < N) split <<= 1;
    return split;
}

FRB_API int frb_selective_scan(const float* xz, int xz_stride, int z_offset, const float* x, const float* low, int low_stride,
                               int b_offset, int c_offset, const float* dt, const float* a_log, const float* d,
                               const int* seq_slot, const int* seq_start, const int* cu_q_len, float* state,
                               long long copy_floats, long long state_offset, void* out, int out_dtype, int num_seqs, int inner,
                               int N, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(N >= 1 && N <= 512, "selective_scan: a state of %d per channel is outside 1..512", N);
    FRB_CHECK_ARG(num_seqs <= 65535, "selective_scan: %d sequences exceed the grid", num_seqs);
    // The most elements a lane (16, 8, 4, 2) that still gives every SM a dozen warps: a lane's work per token beside the
    // updates themselves (its loads, the additions across the lanes, the output) is shared by all of its elements.
    static const int forced = [] { const char* v = getenv("FIELDRUN_B200_SCAN_ELEMENTS"); return v && v[0] ? atoi(v) : 0; }();
    static const int sms = [] { int d = 0, n = 0; cudaGetDevice(&d); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d); return n; }();
    int regs = 2;
    for (int r = 16; r >= 2; r >>= 1)
        if (split_for(N, r) <= 32 && ((long long)num_seqs * inner * split_for(N, r) / 32 >= 12LL * sms || r == 2)) { regs = r; break; }
    if (forced == 2 || forced == 4 || forced == 8 || forced == 16) regs = forced;
    while (split_for(N, regs) > 32) regs <<= 1;              // states of more than 64 elements need more than 2 a lane
    FRB_CHECK_ARG(regs <= 16, "selective_scan: a state of %d per channel is more than the kernel takes", N);
    const int split = split_for(N, regs);
    SelScanParams p;
    p.xz = xz; p.xz_stride = xz_stride; p.z_offset = z_offset; p.x = x; p.low = low; p.low_stride = low_stride;
    p.b_offset = b_offset; p.c_offset = c_offset; p.dt = dt; p.a_log = a_log; p.d = d;
    p.seq = SeqTables{seq_slot, seq_start, cu_q_len};
    p.state = StatePlace{state, copy_floats, state_offset};
    p.out = out; p.inner = inner; p.N = N; p.split = split;
    const int per_block = SEL_BLOCK / split;
    dim3 grid((inner + per_block - 1) / per_block, num_seqs);
    const size_t smem = (size_t)2 * SCAN_TOKENS * N * sizeof(float);
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        if (regs == 2) launch_dependent(selective_scan_kernel<OutT, 2>, grid, dim3(SEL_BLOCK), smem, stream, p);
        else if (regs == 4) launch_dependent(selective_scan_kernel<OutT, 4>, grid, dim3(SEL_BLOCK), smem, stream, p);
        else if (regs == 8) launch_dependent(selective_scan_kernel<OutT, 8>, grid, dim3(SEL_BLOCK), smem, stream, p);
        else launch_dependent(selective_scan_kernel<OutT, 16>, grid, dim3(SEL_BLOCK), smem, stream, p);
    });
    FRB_RETURN_LAUNCH("selective_scan");
}

// ---------------------------------------------------------------------------------------------------- gated_recurrence

struct GatedRecParams {
    const float* yx;         // [T, yx_stride]: the gate branch before bias and activation, channel c at y_offset + c
    const float* y_bias;     // [C] or null
    const float* u;          // [T, C]: the convolution's output
    const float* gates;      // [blocks, T, 2 * bw]: per block the recurrence gate's rows, then the input gate's
    const float* a_bias;     // [C]
    const float* i_bias;     // [C]
    const float* lam;        // [C]
    float* prepared;         // [3][T, C]: the decay less one, the input, the gate branch's activation
    SeqTables seq;
    StatePlace state;        // [C]
    void* out;               // [T, C]
    float gate_constant;
    int yx_stride, y_offset, channels, block_width, num_rows;
};

// First everything that does not depend on the state, for every (row, channel) side by side: the decay less one, the
// gated input and the other branch's activation.  What is left for the pass along the tokens is two multiply-adds a step.
__global__ void __launch_bounds__(128) gated_recurrence_prepare_kernel(GatedRecParams p) {
    after_previous_kernel();
    const int c = blockIdx.y * 128 + threadIdx.x;
    const size_t row = blockIdx.x;
    if (c >= p.channels) return;
    const int bw = p.block_width, blk = c / bw, j = c - blk * bw;
    const float* g_row = p.gates + ((size_t)blk * p.num_rows + row) * 2 * bw + j;
    const float r = sigmoid_f(g_row[0] + p.a_bias[c]), in_gate = sigmoid_f(g_row[bw] + p.i_bias[c]);
    const float log_a = -p.gate_constant * softplus_f(p.lam[c]) * r;
    const size_t at = row * p.channels + c, plane = (size_t)p.num_rows * p.channels;
    p.prepared[at] = expm1f(log_a);
    p.prepared[plane + at] = sqrtf(-expm1f(2.0f * log_a)) * in_gate * p.u[at];          // 1 - a^2 without cancellation
    p.prepared[2 * plane + at] = gelu_tanh_f(p.yx[row * p.yx_stride + p.y_offset + c] + (p.y_bias ? p.y_bias[c] : 0.f));
}

template <typename OutT>
__global__ void __launch_bounds__(128) gated_recurrence_kernel(GatedRecParams p) {
    after_previous_kernel();
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= p.channels) return;
    const int row0 = p.seq.cu_q_len[b], n_tok = p.seq.cu_q_len[b + 1] - row0;
    const int start = p.seq.seq_start[b], slot = p.seq.seq_slot[b];
    const size_t plane = (size_t)p.num_rows * p.channels;
    float S = state_at(p.state, slot, start & 1)[c];
    OutT* out = (OutT*)p.out;
    for (int t0 = 0; t0 < n_tok; t0 += 2 * SCAN_TOKENS) {
        const int count = min(2 * SCAN_TOKENS, n_tok - t0);
        float am1[2 * SCAN_TOKENS], in[2 * SCAN_TOKENS], act[2 * SCAN_TOKENS];
#pragma unroll
        for (int t = 0; t < 2 * SCAN_TOKENS; ++t) {
            const bool has = t < count;
            const size_t at = (size_t)(row0 + t0 + t) * p.channels + c;
            am1[t] = has ? p.prepared[at] : 0.f;
            in[t] = has ? p.prepared[plane + at] : 0.f;
            act[t] = has ? p.prepared[2 * plane + at] : 0.f;
        }
#pragma unroll
        for (int t = 0; t < 2 * SCAN_TOKENS; ++t) {
            if (t < count) {
                S = fmaf(am1[t], S, S) + in[t];
                out[(size_t)(row0 + t0 + t) * p.channels + c] = from_f32<OutT>(S * act[t]);
            }
        }
    }
    state_at(p.state, slot, (start + n_tok) & 1)[c] = S;
}

FRB_API int frb_gated_recurrence(const float* yx, int yx_stride, int y_offset, const float* y_bias, const float* u,
                                 const float* gates, const float* a_bias, const float* i_bias, const float* lam,
                                 float* prepared, const int* seq_slot, const int* seq_start, const int* cu_q_len, float* state,
                                 long long copy_floats, long long state_offset, void* out, int out_dtype, int num_seqs,
                                 int num_rows, int channels, int block_width, float gate_constant, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(num_seqs <= 65535 && (channels + 127) / 128 <= 65535, "gated_recurrence: %d sequences exceed the grid", num_seqs);
    FRB_CHECK_ARG(block_width >= 1 && channels % block_width == 0, "gated_recurrence: %d channels in blocks of %d", channels,
                  block_width);
    GatedRecParams p;
    p.yx = yx; p.yx_stride = yx_stride; p.y_offset = y_offset; p.y_bias = y_bias; p.u = u; p.gates = gates; p.a_bias = a_bias;
    p.i_bias = i_bias; p.lam = lam; p.prepared = prepared; p.seq = SeqTables{seq_slot, seq_start, cu_q_len};
    p.state = StatePlace{state, copy_floats, state_offset};
    p.out = out; p.gate_constant = gate_constant; p.channels = channels; p.block_width = block_width; p.num_rows = num_rows;
    launch_dependent(gated_recurrence_prepare_kernel, dim3(num_rows, (channels + 127) / 128), dim3(128), 0, stream, p);
    dim3 grid((channels + 127) / 128, num_seqs);
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(gated_recurrence_kernel<OutT>, grid, dim3(128), 0, stream, p);
    });
    FRB_RETURN_LAUNCH("gated_recurrence");
}

// ---------------------------------------------------------------------------------------------------- state_space_scan

struct SsdParams {
    const float* proj;       // [T, proj_stride]: z of channel j at z_offset + j, dt of head h at dt_offset + h
    const float* xbc;        // [T, xbc_stride]: x of head h at h * vdim, B of group g at b_offset + g * N, C at c_offset + g * N
    const float* dt_bias;    // [heads]
    const float* a_log;      // [heads]
    const float* d;          // [heads]
    SeqTables seq;
    StatePlace state;        // [heads][N][vdim]
    float* out;              // [T, heads * vdim]: y silu(z), float32 (the norm follows)
    int proj_stride, z_offset, dt_offset, xbc_stride, b_offset, c_offset, heads, vdim, N, groups, parts, npad;
};

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// A block takes (sequence, head, slice of 32 VP value columns); warp `part` keeps NREG rows of the state for each of its
// lane's VP columns (v = lane + 32 j).  Tokens go eight at a time: their B, C, x, z, step and decay lie in one of two
// buffers in shared memory, and while the eight steps of one buffer run (without a barrier; B and C of four rows come
// as one broadcast load of 16 bytes each, for 12 VP multiply-adds) the rows of the next eight tokens are on their way
// into the other (cp.async).  The warps' shares of y are added in warp order.
template <int NREG, int VP>
__global__ void __launch_bounds__(512) state_space_scan_kernel(SsdParams p) {
    extern __shared__ __align__(16) float sm[];
    after_previous_kernel();
    constexpr int COLS = 32 * VP;
    const int N = p.N, npad = p.npad, parts = p.parts, vdim = p.vdim;
    // one buffer: B [SCAN_TOKENS][npad], C [SCAN_TOKENS][npad], x [SCAN_TOKENS][COLS], z [SCAN_TOKENS][COLS], step and decay [SCAN_TOKENS] each
    const int buffer_floats = 2 * SCAN_TOKENS * npad + 2 * SCAN_TOKENS * COLS + 2 * SCAN_TOKENS;
    float* s_y = sm + 2 * buffer_floats;               // [SCAN_TOKENS][parts][COLS]
    const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * COLS;
    const int g = h / (p.heads / p.groups);
    const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
    const int row0 = p.seq.cu_q_len[b], n_tok = p.seq.cu_q_len[b + 1] - row0;
    const int start = p.seq.seq_start[b], slot = p.seq.seq_slot[b];
    const int n0 = part * NREG;
    const float* s_in = state_at(p.state, slot, start & 1) + (size_t)h * N * vdim;
    float S[NREG][VP];
#pragma unroll
    for (int i = 0; i < NREG; ++i)
#pragma unroll
        for (int j = 0; j < VP; ++j) {
            const int v = v0 + lane + 32 * j;
            S[i][j] = (v < vdim && n0 + i < N) ? s_in[(size_t)(n0 + i) * vdim + v] : 0.f;
        }
    const float dt_bias = p.dt_bias[h], rate = expf(p.a_log[h]), dskip = p.d[h];
    for (int i = threadIdx.x; i < 2 * buffer_floats; i += blockDim.x) sm[i] = 0.f;      // the padding stays zero
    __syncthreads();
    const int chunks = (n_tok + SCAN_TOKENS - 1) / SCAN_TOKENS;

    // asks for the rows of chunk `k` into its buffer; the step and the decay are made here and stored directly
    auto stage = [&](int k) {
        float* s_b = sm + (k & 1) * buffer_floats;
        float* s_c = s_b + SCAN_TOKENS * npad;
        float* s_x = s_c + SCAN_TOKENS * npad;
        float* s_z = s_x + SCAN_TOKENS * COLS;
        float* s_dt = s_z + SCAN_TOKENS * COLS;
        const int t0 = k * SCAN_TOKENS, count = min(SCAN_TOKENS, n_tok - t0);
        for (int i = threadIdx.x; i < count * N; i += blockDim.x) {
            const int t = i / N, n = i - t * N;
            const float* row = p.xbc + (size_t)(row0 + t0 + t) * p.xbc_stride;
            copy_async4(s_b + t * npad + n, row + p.b_offset + g * N + n);
            copy_async4(s_c + t * npad + n, row + p.c_offset + g * N + n);
        }
        for (int i = threadIdx.x; i < count * COLS; i += blockDim.x) {
            const int t = i / COLS, l = i - t * COLS;
            if (v0 + l < vdim) {
                const size_t row = (size_t)(row0 + t0 + t);
                copy_async4(s_x + i, p.xbc + row * p.xbc_stride + h * vdim + v0 + l);
                copy_async4(s_z + i, p.proj + row * p.proj_stride + p.z_offset + h * vdim + v0 + l);
            }
        }
        if (threadIdx.x < count) {
            const float step = softplus_f(p.proj[(size_t)(row0 + t0 + threadIdx.x) * p.proj_stride + p.dt_offset + h] + dt_bias);
            s_dt[threadIdx.x] = step;
            s_dt[SCAN_TOKENS + threadIdx.x] = decay_less_one(-rate * step);
        }
    };

    if (chunks > 0) stage(0);
    for (int k = 0; k < chunks; ++k) {
        const int t0 = k * SCAN_TOKENS, count = min(SCAN_TOKENS, n_tok - t0);
        copies_wait();
        __syncthreads();                               // chunk k lies in its buffer; nobody reads the other one any more
        if (k + 1 < chunks) stage(k + 1);
        const float* s_b = sm + (k & 1) * buffer_floats;
        const float* s_c = s_b + SCAN_TOKENS * npad;
        const float* s_x = s_c + SCAN_TOKENS * npad;
        const float* s_z = s_x + SCAN_TOKENS * COLS;
        const float* s_dt = s_z + SCAN_TOKENS * COLS;
        const float* s_a = s_dt + SCAN_TOKENS;
#pragma unroll
        for (int t = 0; t < SCAN_TOKENS; ++t) {
            if (t < count) {
                const float am1 = s_a[t], step = s_dt[t];
                float sx[VP], y[VP];
#pragma unroll
                for (int j = 0; j < VP; ++j) { sx[j] = step * s_x[t * COLS + lane + 32 * j]; y[j] = 0.f; }
#pragma unroll
                for (int i = 0; i < NREG; i += 4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(s_b + t * npad + n0 + i);
                    const float4 c4 = *reinterpret_cast<const float4*>(s_c + t * npad + n0 + i);
                    const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int j = 0; j < VP; ++j) {
                            S[i + q][j] = fmaf(am1, S[i + q][j], S[i + q][j]) + bb[q] * sx[j];
                            y[j] = fmaf(S[i + q][j], cc[q], y[j]);
                        }
                }
#pragma unroll
                for (int j = 0; j < VP; ++j) s_y[(t * parts + part) * COLS + lane + 32 * j] = y[j];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < count * COLS; i += blockDim.x) {
            const int t = i / COLS, l = i - t * COLS;
            if (v0 + l < vdim) {
                float y = 0.f;
                for (int q = 0; q < parts; ++q) y += s_y[(t * parts + q) * COLS + l];
                p.out[(size_t)(row0 + t0 + t) * (size_t)(p.heads * vdim) + h * vdim + v0 + l] = (y + dskip * s_x[i]) * silu_f(s_z[i]);
            }
        }
    }
    float* s_out = state_at(p.state, slot, (start + n_tok) & 1) + (size_t)h * N * vdim;
#pragma unroll
    for (int i = 0; i < NREG; ++i)
#pragma unroll
        for (int j = 0; j < VP; ++j) {
            const int v = v0 + lane + 32 * j;
            if (v < vdim && n0 + i < N) s_out[(size_t)(n0 + i) * vdim + v] = S[i][j];
        }
}

FRB_API int frb_state_space_scan(const float* proj, int proj_stride, int z_offset, int dt_offset, const float* xbc,
                                 int xbc_stride, int b_offset, int c_offset, const float* dt_bias, const float* a_log,
                                 const float* d, const int* seq_slot, const int* seq_start, const int* cu_q_len, float* state,
                                 long long copy_floats, long long state_offset, float* out, int num_seqs, int heads, int vdim,
                                 int N, int groups, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(groups >= 1 && heads % groups == 0, "state_space_scan: %d heads are not a multiple of %d groups", heads, groups);
    FRB_CHECK_ARG(N >= 1 && N <= 1024, "state_space_scan: a state of %d rows per head is outside 1..1024", N);
    int nreg = 8;
    while ((N + nreg - 1) / nreg > 16) nreg <<= 1;
    // value columns a lane: as many as the head has (in 32s) while a thread's share of the state stays within 64 registers
    int vp = vdim > 64 ? 4 : vdim > 32 ? 2 : 1;
    while (vp > 1 && nreg * vp > 64) vp >>= 1;
    const int cols = 32 * vp;
    FRB_CHECK_ARG(heads <= 65535 && (vdim + cols - 1) / cols <= 65535, "state_space_scan: %d heads of %d exceed the grid", heads, vdim);
    SsdParams p;
    p.proj = proj; p.proj_stride = proj_stride; p.z_offset = z_offset; p.dt_offset = dt_offset; p.xbc = xbc;
    p.xbc_stride = xbc_stride; p.b_offset = b_offset; p.c_offset = c_offset; p.dt_bias = dt_bias; p.a_log = a_log; p.d = d;
    p.seq = SeqTables{seq_slot, seq_start, cu_q_len};
    p.state = StatePlace{state, copy_floats, state_offset};
    p.out = out; p.heads = heads; p.vdim = vdim; p.N = N; p.groups = groups;
    p.parts = (N + nreg - 1) / nreg;
    p.npad = p.parts * nreg;
    const size_t smem = (2 * ((size_t)2 * SCAN_TOKENS * p.npad + 2 * SCAN_TOKENS * cols + 2 * SCAN_TOKENS)
                         + (size_t)SCAN_TOKENS * p.parts * cols) * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "state_space_scan: a state of %d rows needs more shared memory than a block has", N);
    dim3 grid(num_seqs, heads, (vdim + cols - 1) / cols);
    dim3 block(32 * p.parts);
#define FRB_SSD(NREG, VP)                                                                                            \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(state_space_scan_kernel<NREG, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_dependent(state_space_scan_kernel<NREG, VP>, grid, block, smem, stream, p);                           \
    } while (0)
    if (nreg == 8) { if (vp == 4) FRB_SSD(8, 4); else if (vp == 2) FRB_SSD(8, 2); else FRB_SSD(8, 1); }
    else if (nreg == 16) { if (vp == 4) FRB_SSD(16, 4); else if (vp == 2) FRB_SSD(16, 2); else FRB_SSD(16, 1); }
    else if (nreg == 32) { if (vp == 2) FRB_SSD(32, 2); else FRB_SSD(32, 1); }
    else FRB_SSD(64, 1);
#undef FRB_SSD
    FRB_RETURN_LAUNCH("state_space_scan");
}

// ---------------------------------------------------------------------------------------------------- group_rms_norm

template <typename OutT>
__global__ void __launch_bounds__(128) group_rms_norm_kernel(const float* __restrict__ in, const float* __restrict__ weight,
                                                             OutT* __restrict__ out, int width, int part, float eps) {
    __shared__ float scratch[32];
    after_previous_kernel();
    const size_t base = (size_t)blockIdx.x * width + (size_t)blockIdx.y * part;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += 128) {
        const float v = in[base + i];
        ss += v * v;
    }
    ss = block_sum<128>(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += 128)
        out[base + i] = from_f32<OutT>(in[base + i] * rinv * weight[blockIdx.y * part + i]);
}

FRB_API int frb_group_rms_norm(const float* in, const float* weight, void* out, int out_dtype, int num_rows, int width,
                               int norm_groups, float eps, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(norm_groups >= 1 && width % norm_groups == 0 && norm_groups <= 65535,
                  "group_rms_norm: a row of %d in %d parts", width, norm_groups);
    dim3 grid(num_rows, norm_groups);
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(group_rms_norm_kernel<OutT>, grid, dim3(128), 0, stream, in, weight, (OutT*)out, width,
                         width / norm_groups, eps);
    });
    FRB_RETURN_LAUNCH("group_rms_norm");
}

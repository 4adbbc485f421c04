// Recurrent mixers: a minGRU and a gated linear recurrence behind a short causal
// convolution. The state of a request lives in float32 in its slot, `state[slot]`, and
// every kernel here runs a step's tokens of sequence s (rows q_start[s] .. q_start[s+1]-1
// of the batch) in order from the state the step before left. Gates, decays and the state
// are float32 in both engines; only the output (the input of the next product) is stored
// in the activation type. One thread owns one channel, so a channel's arithmetic is the
// same however the tokens were cut into steps.
#include "common.cuh"

namespace mb {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ---- the scan ----------------------------------------------------------------------------
// Both recurrences are S_t = a_t S_{t-1} + b_t per channel, with a_t, b_t read off the
// token alone. A block takes blockDim.x channels of one sequence (8 when the step is cut
// into runs, so that a long prompt spreads over many SMs; 32 for a decode step) and cuts the
// step's tokens into blockDim.y runs (up to 64): every thread first folds its run into (A, B) with S_end = A S_start + B,
// one thread per channel chains the runs' starts, and every thread then walks its run again
// from its start and writes the outputs. The state that goes on to the next step is the
// last run's own final value. A decode step (one token) is a single run.
constexpr int SC_CHANNELS = 32;
constexpr int SC_MAX_RUNS = 64;

template <typename T, typename F>
__device__ __forceinline__ void scan_runs(const F& f, float* cell, int begin, int end, int c,
                                          bool live, T* __restrict__ out, int width) {
    __shared__ float run_a[SC_MAX_RUNS][SC_CHANNELS], run_b[SC_MAX_RUNS][SC_CHANNELS];
    const int runs = blockDim.y, k = threadIdx.y, x = threadIdx.x;
    const int n = end - begin;
    const int len = (n + runs - 1) / runs;
    const int t0 = min(end, begin + k * len), t1 = min(end, t0 + len);
    if (runs > 1) {
        float A = 1.f, B = 0.f;
        if (live) {
#pragma unroll 4
            for (int t = t0; t < t1; ++t) {
                float a, b, o;
                f(t, c, a, b, o, false);      // the output's gate is not needed for the fold
                B = a * B + b;
                A *= a;
            }
        }
        run_a[k][x] = A;
        run_b[k][x] = B;
        __syncthreads();
        if (k == 0 && live) {
            float s = *cell;
            for (int j = 0; j < runs; ++j) {
                const float A2 = run_a[j][x], B2 = run_b[j][x];
                run_a[j][x] = s;                 // the run's start
                s = A2 * s + B2;
            }
        }
        __syncthreads();
    }
    if (!live || t0 >= t1) return;
    float s = runs > 1 ? run_a[k][x] : *cell;
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float a, b, o;
        f(t, c, a, b, o, true);
        s = a * s + b;
        out[(int64_t)t * width + c] = from_float<T>(s * o);
    }
    if (t1 == end) *cell = s;
}

// pre: [tokens][3 * width] float32 = [gate z | candidate u | output gate g] before their
// activations. S <- (1 - z) S + z c with z = sigmoid(.), c = u + 1/2 (u >= 0) or sigmoid(u);
// out = S * silu(g).
struct MinGruStep {
    const float* pre;
    int width;
    __device__ __forceinline__ void operator()(int t, int c, float& a, float& b, float& o,
                                               bool with_gate) const {
        // read-only loads: they may move ahead of the stores of the tokens before
        const float* row = pre + (int64_t)t * 3 * width;
        const float z = sigmoid_f(__ldg(row + c));
        const float u = __ldg(row + width + c);
        a = 1.f - z;
        b = z * (u >= 0.f ? u + 0.5f : sigmoid_f(u));
        o = 0.f;
        if (with_gate) {
            const float g = __ldg(row + 2 * width + c);
            o = g * sigmoid_f(g);
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(1024)
mingru_scan_kernel(const float* __restrict__ pre, float* __restrict__ state,
                   const int* __restrict__ q_start, const int* __restrict__ slots,
                   T* __restrict__ out, int width) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (begin >= end) return;
    const bool live = c < width;
    MinGruStep f{pre, width};
    scan_runs<T>(f, state + (int64_t)slots[seq] * width + (live ? c : 0), begin, end, c, live, out, width);
}

// u[t][c] = sum_k taps_w[c][k] * x[t - (taps - 1 - k)][c] + bias[c], x = pre[:, offset + c]
// (row stride ld). Inputs from before this step come from the state: state[slot][j][c] is
// the input j tokens before the step's first token (j = 1 .. taps - 1; zero before the
// sequence began, because a fresh slot is zeroed). The state is not changed here.
__global__ void causal_conv_kernel(const float* __restrict__ pre, int ld, int offset,
                                   const float* __restrict__ taps_w, const float* __restrict__ bias,
                                   const float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ slots, const int* __restrict__ seq_of_token,
                                   float* __restrict__ u, int width, int taps) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    const int seq = seq_of_token[t];
    if (c >= width || seq < 0) return;
    const int begin = q_start[seq];
    const int at = t - begin;
    const float* past = state + (int64_t)slots[seq] * taps * width;
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int src = at - (taps - 1 - k);
        const float x = src >= 0 ? pre[(int64_t)(begin + src) * ld + offset + c]
                                 : past[(int64_t)(-src) * width + c];
        acc = fmaf(taps_w[c * taps + k], x, acc);
    }
    u[(int64_t)t * width + c] = acc + bias[c];
}

// gates[t][kind * width + b * size + o] = sigmoid(sum_i w[kind][b][i][o] * u[t][b * size + i]
// + bias[kind][b][o]) for the two kinds of gate (r, i): block-diagonal products in float32
// FMAs, the weights held input-major so that consecutive threads (outputs o) read
// consecutive addresses. A block computes 128 outputs of one block b, both kinds (they read
// the same inputs), for BG_TOKENS tokens (32 in a prompt step, 8 in a decode step), the inputs
// staged token-minor so that four tokens come with one shared-memory load; i ascends, so the
// order of each sum is fixed.
template <int BG_TOKENS>
__global__ void __launch_bounds__(128)
block_gates_kernel(const float* __restrict__ u, const float* __restrict__ w,
                   const float* __restrict__ bias, float* __restrict__ gates, int tokens, int width,
                   int blocks, int size) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float u_s[];          // [size][BG_TOKENS]
    const int per = (size + 127) / 128;                  // output tiles per block b
    const int otile = blockIdx.x % per;
    const int b = blockIdx.x / per;
    const int t0 = blockIdx.y * BG_TOKENS;
    for (int idx = threadIdx.x; idx < BG_TOKENS * size; idx += blockDim.x) {
        const int tt = idx / size, i = idx - tt * size;
        u_s[i * BG_TOKENS + tt] = t0 + tt < tokens ? u[(int64_t)(t0 + tt) * width + b * size + i] : 0.f;
    }
    __syncthreads();
    const int o = otile * 128 + threadIdx.x;
    if (o >= size) return;
    const float* wr = w + ((int64_t)b * size) * size + o;                    // kind 0
    const float* wi = w + ((int64_t)(blocks + b) * size) * size + o;         // kind 1
    float ar[BG_TOKENS], ai[BG_TOKENS];
#pragma unroll
    for (int tt = 0; tt < BG_TOKENS; ++tt) ar[tt] = ai[tt] = 0.f;
#pragma unroll 4
    for (int i = 0; i < size; ++i) {
        const float vr = wr[(int64_t)i * size], vi = wi[(int64_t)i * size];
        const float4* row = reinterpret_cast<const float4*>(u_s + i * BG_TOKENS);
#pragma unroll
        for (int q = 0; q < BG_TOKENS / 4; ++q) {
            const float4 x = row[q];
            ar[4 * q] = fmaf(vr, x.x, ar[4 * q]);
            ar[4 * q + 1] = fmaf(vr, x.y, ar[4 * q + 1]);
            ar[4 * q + 2] = fmaf(vr, x.z, ar[4 * q + 2]);
            ar[4 * q + 3] = fmaf(vr, x.w, ar[4 * q + 3]);
            ai[4 * q] = fmaf(vi, x.x, ai[4 * q]);
            ai[4 * q + 1] = fmaf(vi, x.y, ai[4 * q + 1]);
            ai[4 * q + 2] = fmaf(vi, x.z, ai[4 * q + 2]);
            ai[4 * q + 3] = fmaf(vi, x.w, ai[4 * q + 3]);
        }
    }
    const float br = bias[b * size + o], bi = bias[(blocks + b) * size + o];
#pragma unroll
    for (int tt = 0; tt < BG_TOKENS; ++tt)
        if (t0 + tt < tokens) {
            float* row = gates + (int64_t)(t0 + tt) * 2 * width + b * size + o;
            row[0] = sigmoid_f(ar[tt] + br);
            row[width] = sigmoid_f(ai[tt] + bi);
        }
}

// The same for the few tokens of a decode step, where the gate matrices have to be streamed
// once and few blocks would do it slowly: a block computes 32 outputs (both kinds) of one
// block b for up to 8 tokens, its four warps each taking a quarter of the inputs i; the
// quarters are added in a fixed order through shared memory.
__global__ void __launch_bounds__(128)
block_gates_few_kernel(const float* __restrict__ u, const float* __restrict__ w,
                       const float* __restrict__ bias, float* __restrict__ gates, int tokens,
                       int width, int blocks, int size) {
    grid_dependency_sync();
    extern __shared__ __align__(16) float fs[];            // u: [size][8], then partial sums
    float* u_s = fs;
    float* part = fs + size * 8;                            // [4][2][8][32]
    const int per = (size + 31) / 32;
    const int otile = blockIdx.x % per;
    const int b = blockIdx.x / per;
    const int t0 = blockIdx.y * 8;
    for (int idx = threadIdx.x; idx < 8 * size; idx += blockDim.x) {
        const int tt = idx / size, i = idx - tt * size;
        u_s[i * 8 + tt] = t0 + tt < tokens ? u[(int64_t)(t0 + tt) * width + b * size + i] : 0.f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int o = otile * 32 + lane;
    const int quarter = (size + 3) / 4;
    const int i0 = slice * quarter, i1 = min(size, i0 + quarter);
    float ar[8], ai[8];
#pragma unroll
    for (int tt = 0; tt < 8; ++tt) ar[tt] = ai[tt] = 0.f;
    if (o < size) {
        const float* wr = w + ((int64_t)b * size) * size + o;
        const float* wi = w + ((int64_t)(blocks + b) * size) * size + o;
#pragma unroll 8
        for (int i = i0; i < i1; ++i) {
            const float vr = __ldg(wr + (int64_t)i * size), vi = __ldg(wi + (int64_t)i * size);
            const float4 x0 = *reinterpret_cast<const float4*>(u_s + i * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(u_s + i * 8 + 4);
            ar[0] = fmaf(vr, x0.x, ar[0]); ar[1] = fmaf(vr, x0.y, ar[1]);
            ar[2] = fmaf(vr, x0.z, ar[2]); ar[3] = fmaf(vr, x0.w, ar[3]);
            ar[4] = fmaf(vr, x1.x, ar[4]); ar[5] = fmaf(vr, x1.y, ar[5]);
            ar[6] = fmaf(vr, x1.z, ar[6]); ar[7] = fmaf(vr, x1.w, ar[7]);
            ai[0] = fmaf(vi, x0.x, ai[0]); ai[1] = fmaf(vi, x0.y, ai[1]);
            ai[2] = fmaf(vi, x0.z, ai[2]); ai[3] = fmaf(vi, x0.w, ai[3]);
            ai[4] = fmaf(vi, x1.x, ai[4]); ai[5] = fmaf(vi, x1.y, ai[5]);
            ai[6] = fmaf(vi, x1.z, ai[6]); ai[7] = fmaf(vi, x1.w, ai[7]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < 8; ++tt) {
        part[((slice * 2 + 0) * 8 + tt) * 32 + lane] = ar[tt];
        part[((slice * 2 + 1) * 8 + tt) * 32 + lane] = ai[tt];
    }
    __syncthreads();
    // 2 kinds x 8 tokens x 32 outputs = 512 results, four per thread
    for (int idx = threadIdx.x; idx < 2 * 8 * 32; idx += blockDim.x) {
        const int l = idx & 31, tt = (idx >> 5) & 7, kind = idx >> 8;
        const int oo = otile * 32 + l;
        if (oo >= size || t0 + tt >= tokens) continue;
        float v = 0.f;
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) v += part[((sl * 2 + kind) * 8 + tt) * 32 + l];
        v += bias[(kind * blocks + b) * size + oo];
        gates[(int64_t)(t0 + tt) * 2 * width + kind * width + b * size + oo] = sigmoid_f(v);
    }
}

// pre: [tokens][2 * width] float32 = [branch y | convolution input x]; u: the convolution's
// output; gates: [tokens][2 * width] = [r | i] after their sigmoids.
// a = exp(-decay_scale * r * softplus_lam), S <- a S + sqrt(1 - a^2) * i * u, out = S * gelu(y).
// state[slot]: row 0 = S, row j = the convolution's input j tokens back; the rows 1.. are
// brought up to the end of this step here, after every token's convolution has been taken.
struct GatedStep {
    const float* pre;
    const float* u;
    const float* gates;
    const float* softplus_lam;
    float decay_scale;
    int width;
    __device__ __forceinline__ void operator()(int t, int c, float& a, float& b, float& o,
                                               bool with_gate) const {
        const float r = __ldg(gates + (int64_t)t * 2 * width + c);
        const float i = __ldg(gates + (int64_t)t * 2 * width + width + c);
        const float x = __ldg(u + (int64_t)t * width + c);
        a = expf(-decay_scale * r * __ldg(softplus_lam + c));
        b = sqrtf(1.f - a * a) * i * x;
        o = with_gate ? gelu_tanh_f(__ldg(pre + (int64_t)t * 2 * width + c)) : 0.f;
    }
};

template <typename T>
__global__ void __launch_bounds__(1024)
gated_recurrence_scan_kernel(const float* __restrict__ pre, const float* __restrict__ u,
                             const float* __restrict__ gates, const float* __restrict__ softplus_lam,
                             float decay_scale, float* __restrict__ state,
                             const int* __restrict__ q_start, const int* __restrict__ slots,
                             T* __restrict__ out, int width, int taps) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (begin >= end) return;
    const bool live = c < width;
    float* mine = state + (int64_t)slots[seq] * taps * width + (live ? c : 0);
    if (live && threadIdx.y == 0) {
        const int n = end - begin;
        float old[16];
        for (int j = 1; j < taps; ++j) old[j] = mine[(int64_t)j * width];
        for (int j = 1; j < taps; ++j) {
            const int idx = n - j;
            mine[(int64_t)j * width] =
                idx >= 0 ? pre[(int64_t)(begin + idx) * 2 * width + width + c] : old[j - n];
        }
    }
    GatedStep f{pre, u, gates, softplus_lam, decay_scale, width};
    scan_runs<T>(f, mine, begin, end, c, live, out, width);
}

}  // namespace mb

using namespace mb;

// Runs per sequence for a step whose longest portion has `max_q_len` tokens: about 16
// tokens per run, at most SC_MAX_RUNS (with 8 channels a block: 512 threads).
static int scan_run_count(int max_q_len) {
    int runs = (max_q_len + 15) / 16;
    return runs < 1 ? 1 : (runs > SC_MAX_RUNS ? SC_MAX_RUNS : runs);
}

MB_EXPORT int mb_mingru_scan(const float* pre, float* state, const int* q_start, const int* slots,
                             void* out, int num_seqs, int max_q_len, int width, int dtype,
                             void* stream) {
    if (num_seqs <= 0 || width <= 0) return MB_OK;
    if (num_seqs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    const int runs = scan_run_count(max_q_len);
    const int channels = runs > 1 ? 8 : SC_CHANNELS;
    dim3 grid((width + channels - 1) / channels, num_seqs);
    dim3 block(channels, runs);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((mingru_scan_kernel<float>), grid, block, 0, s, pre, state, q_start, slots, (float*)out, width);
    else if (dtype == MB_BF16)
        MB_LAUNCH((mingru_scan_kernel<__nv_bfloat16>), grid, block, 0, s, pre, state, q_start, slots,
                  (__nv_bfloat16*)out, width);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

MB_EXPORT int mb_causal_conv(const float* pre, int ld, int offset, const float* taps_w,
                             const float* bias, const float* state, const int* q_start,
                             const int* slots, const int* seq_of_token, float* u, int tokens,
                             int width, int taps, void* stream) {
    if (tokens <= 0 || width <= 0) return MB_OK;
    if (taps < 1 || taps > 16 || tokens > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid((width + 127) / 128, tokens);
    MB_LAUNCH((causal_conv_kernel), grid, 128, 0, (cudaStream_t)stream, pre, ld, offset, taps_w, bias,
              state, q_start, slots, seq_of_token, u, width, taps);
    return launch_status();
}

// w: [kinds][blocks][size (in)][size (out)] float32; bias: [kinds][blocks][size].
MB_EXPORT int mb_block_gates(const float* u, const float* w, const float* bias, float* gates,
                             int tokens, int width, int blocks, int kinds, void* stream) {
    if (tokens <= 0 || width <= 0) return MB_OK;
    if (blocks <= 0 || width % blocks || kinds != 2) return MB_ERR_UNSUPPORTED_SIZE;
    const int size = width / blocks;
    const bool few = tokens <= 16;
    const int tile = few ? 8 : 32;
    const size_t smem = (size_t)tile * size * sizeof(float) + (few ? 4 * 2 * 8 * 32 * sizeof(float) : 0);
    if (smem > 200 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    static size_t raised[2] = {0, 0};
    size_t& mine = raised[few ? 0 : 1];
    if (smem > 48 * 1024 && smem > mine) {
        const cudaError_t rc = few
            ? cudaFuncSetAttribute(block_gates_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
            : cudaFuncSetAttribute(block_gates_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc != cudaSuccess) return MB_ERR_UNSUPPORTED_SIZE;
        mine = smem;
    }
    const int rows = (tokens + tile - 1) / tile;
    if (rows > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (few) {
        dim3 grid(((size + 31) / 32) * blocks, rows);
        MB_LAUNCH((block_gates_few_kernel), grid, 128, smem, (cudaStream_t)stream, u, w, bias, gates,
                  tokens, width, blocks, size);
    } else {
        dim3 grid(((size + 127) / 128) * blocks, rows);
        MB_LAUNCH((block_gates_kernel<32>), grid, 128, smem, (cudaStream_t)stream, u, w, bias, gates,
                  tokens, width, blocks, size);
    }
    return launch_status();
}

MB_EXPORT int mb_gated_recurrence_scan(const float* pre, const float* u, const float* gates,
                                       const float* softplus_lam, float decay_scale, float* state,
                                       const int* q_start, const int* slots, void* out,
                                       int num_seqs, int max_q_len, int width, int taps, int dtype,
                                       void* stream) {
    if (num_seqs <= 0 || width <= 0) return MB_OK;
    if (taps < 1 || taps > 16 || num_seqs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    const int runs = scan_run_count(max_q_len);
    const int channels = runs > 1 ? 8 : SC_CHANNELS;
    dim3 grid((width + channels - 1) / channels, num_seqs);
    dim3 block(channels, runs);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((gated_recurrence_scan_kernel<float>), grid, block, 0, s, pre, u, gates, softplus_lam,
                  decay_scale, state, q_start, slots, (float*)out, width, taps);
    else if (dtype == MB_BF16)
        MB_LAUNCH((gated_recurrence_scan_kernel<__nv_bfloat16>), grid, block, 0, s, pre, u, gates,
                  softplus_lam, decay_scale, state, q_start, slots, (__nv_bfloat16*)out, width, taps);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

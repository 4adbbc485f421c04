// Mixers whose memory is a matrix per head: a Mamba-2 state-space layer and a gated delta
// rule, with the short causal convolution in front of them and the gated group norm behind.
// A request's state lives in float32 in its slot: `cells` (the heads' matrices) and `tail`
// (the convolution's last taps - 1 inputs) are two regions of one state row, so both come
// as a pointer plus the distance between two slots' rows. Every kernel runs a step's tokens
// of sequence s (rows q_start[s] .. q_start[s+1]-1) in order from the state the step before
// left. Everything here is float32 in both engines; only the group norm's output (the input
// of the output projection) is stored in the activation type.
//
// Work split of the two scans: a block takes one head of one sequence (and a range of the
// head's columns p); inside a warp four columns are held by eight lanes each, lane `slice`
// keeping the matrix rows slice, slice + 8, slice + 16, ... of its column in registers. A
// token's read-out is a sum over rows: partial sums per lane, then three shuffles. The
// tokens' inputs are staged through shared memory sixteen tokens at a time, so the block
// meets once per sixteen tokens. A column's arithmetic is the same however the tokens were
// cut into steps.
//
// The template parameter S is the type the matrix is held in while a step runs. A float32
// matrix that takes in a thousand tokens one by one gathers a rounding error of some 1e-6 of
// its size, which is small beside bfloat16 activations and is what the bfloat16 engine runs
// with; the float32 engine holds the matrix and its sums in double inside a step (S =
// double) and rounds to float32 only when the step's last token is in, so a long prompt
// costs one rounding where it would cost one per token. The decay that multiplies the matrix
// at every token is computed in double in both and rounded once: an error of an ulp in expf
// that leans one way grows linearly with the number of tokens a contribution has to survive.
// Between steps the state is float32 in both.
#include "common.cuh"

namespace mb {

constexpr int SS_TILE = 16;      // tokens staged at a time
constexpr int SS_SLICES = 8;     // lanes that share a column

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__device__ __forceinline__ float slice_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

__device__ __forceinline__ double softplus_f(double x) { return x > 40.0 ? x : log1p(exp(x)); }

__device__ __forceinline__ double slice_sum(double v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

// ---- short causal convolution --------------------------------------------------------------
// out[t][c] = act(sum_k w[c][k] * x[t - (taps - 1 - k)][c] + bias[c]), x = pre[:, offset + c]
// (row stride ld). Inputs from before the step come from the tail: tail[slot][(j - 1) *
// channels + c] is the input j tokens before the step's first token (zero before the
// sequence began, because a fresh slot is zeroed). The tail is not changed here.
__global__ void conv_act_kernel(const float* __restrict__ pre, int ld, int offset,
                                const float* __restrict__ w, const float* __restrict__ bias,
                                const float* __restrict__ tail, int64_t tail_stride,
                                const int* __restrict__ q_start, const int* __restrict__ slots,
                                const int* __restrict__ seq_of_token, float* __restrict__ out,
                                int channels, int taps, int act) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    const int seq = seq_of_token[t];
    if (c >= channels || seq < 0) return;
    const int begin = q_start[seq];
    const int at = t - begin;
    const float* past = tail + (int64_t)slots[seq] * tail_stride;
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int src = at - (taps - 1 - k);
        const float x = src >= 0 ? pre[(int64_t)(begin + src) * ld + offset + c]
                                 : past[(int64_t)(-src - 1) * channels + c];
        acc = fmaf(w[c * taps + k], x, acc);
    }
    if (bias) acc += bias[c];
    if (act == 1) acc = silu_f(acc);
    out[(int64_t)t * channels + c] = acc;
}

// The tail after the step: the last taps - 1 inputs of (old tail, this step's inputs). Runs
// after every token's convolution has been taken.
__global__ void conv_tail_update_kernel(const float* __restrict__ pre, int ld, int offset,
                                        float* __restrict__ tail, int64_t tail_stride,
                                        const int* __restrict__ q_start,
                                        const int* __restrict__ slots, int channels, int taps) {
    grid_dependency_sync();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], n = q_start[seq + 1] - begin;
    if (c >= channels || n <= 0) return;
    float* mine = tail + (int64_t)slots[seq] * tail_stride + c;
    float old[16];
    for (int j = 1; j < taps; ++j) old[j] = mine[(int64_t)(j - 1) * channels];
    for (int j = 1; j < taps; ++j) {
        const int idx = n - j;
        mine[(int64_t)(j - 1) * channels] =
            idx >= 0 ? pre[(int64_t)(begin + idx) * ld + offset + c] : old[j - n];
    }
}

// ---- Mamba-2 -------------------------------------------------------------------------------
// xbc: [tokens][inner + 2 * groups * n_state] = [x | B | C] behind convolution and SiLU;
// pre[:, dt_offset + head] the raw step sizes. Per head, with B and C of the head's group:
//   dt = softplus(raw + dt_bias);  S <- exp(neg_rate * dt) S + dt * B x^T;  y = S^T C + skip * x
// S is [n_state][vdim] at cells[slot][(head * n_state + n) * vdim + p].
template <int NPT, typename S>
__global__ void __launch_bounds__(512)
mamba2_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ pre, int pre_ld,
                   int dt_offset, const float* __restrict__ dt_bias,
                   const float* __restrict__ neg_rate, const float* __restrict__ skip,
                   float* __restrict__ cells, int64_t cell_stride, const int* __restrict__ q_start,
                   const int* __restrict__ slots, float* __restrict__ y, int heads, int vdim,
                   int n_state, int groups, int chunks_per_head) {
    grid_dependency_sync();
    extern __shared__ float sm[];
    constexpr int NP = NPT * SS_SLICES;
    const int cols = (blockDim.x >> 5) * 4;
    float* b_s = sm;                          // [SS_TILE][NP]
    float* c_s = b_s + SS_TILE * NP;          // [SS_TILE][NP]
    float* x_s = c_s + SS_TILE * NP;          // [SS_TILE][cols]
    __shared__ S dt_s[SS_TILE], da_s[SS_TILE];
    const int head = blockIdx.x / chunks_per_head, chunk = blockIdx.x - head * chunks_per_head;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (begin >= end) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int slice = lane & 7, p_local = warp * 4 + (lane >> 3);
    const int p = chunk * cols + p_local;
    const bool live = p < vdim;
    const int inner = heads * vdim, width = inner + 2 * groups * n_state;
    const int g = head / (heads / groups);
    float* mine = cells + (int64_t)slots[seq] * cell_stride + (int64_t)head * n_state * vdim;
    S s[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = slice + SS_SLICES * i;
        s[i] = (live && n < n_state) ? (S)mine[(int64_t)n * vdim + p] : (S)0;
    }
    const float rate = neg_rate[head], bias = dt_bias[head], d_skip = skip[head];
    for (int t0 = begin; t0 < end; t0 += SS_TILE) {
        const int nt = min(SS_TILE, end - t0);
        __syncthreads();                      // the tile before is consumed
        for (int idx = tid; idx < nt * NP; idx += blockDim.x) {
            const int tt = idx / NP, n = idx - tt * NP;
            const float* row = xbc + (int64_t)(t0 + tt) * width + inner + g * n_state;
            b_s[idx] = n < n_state ? row[n] : 0.f;
            c_s[idx] = n < n_state ? row[groups * n_state + n] : 0.f;
        }
        for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
            const int tt = idx / cols, pl = idx - tt * cols;
            const int pp = chunk * cols + pl;
            x_s[idx] = pp < vdim ? xbc[(int64_t)(t0 + tt) * width + head * vdim + pp] : 0.f;
        }
        if (tid < nt) {
            // in double whatever S is: sixteen numbers a tile, and the decay comes out rounded
            // to nearest instead of leaning one way
            const double dt = softplus_f((double)pre[(int64_t)(t0 + tid) * pre_ld + dt_offset + head] +
                                         (double)bias);
            dt_s[tid] = (S)dt;
            da_s[tid] = (S)exp((double)rate * dt);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float x = x_s[tt * cols + p_local];
            const S da = da_s[tt];
            const S dtx = dt_s[tt] * (S)x;
            const float* bt = b_s + tt * NP + slice;
            const float* ct = c_s + tt * NP + slice;
            S acc = (S)0;
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                s[i] = fma(da, s[i], dtx * (S)bt[SS_SLICES * i]);
                acc = fma(s[i], (S)ct[SS_SLICES * i], acc);
            }
            acc = slice_sum(acc);
            if (slice == 0 && live)
                y[(int64_t)(t0 + tt) * inner + head * vdim + p] = (float)fma((S)d_skip, (S)x, acc);
        }
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = slice + SS_SLICES * i;
        if (live && n < n_state) mine[(int64_t)n * vdim + p] = (float)s[i];
    }
}

// ---- gated delta rule ------------------------------------------------------------------------
// qkv: [tokens][2 * key_heads * dim + heads * vdim] = [q | k | v] behind convolution and SiLU;
// pre[:, beta_offset + head] and pre[:, decay_offset + head] the raw gate inputs. Head h
// reads q/k head h / (heads / key_heads). Per head:
//   q <- q / sqrt(sum q^2 + unit_eps) * dim^-1/2;  k <- k / sqrt(sum k^2 + unit_eps)
//   beta = sigmoid(raw_b);  g = exp(neg_rate * softplus(raw_a + dt_bias))
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// computed from the matrix as the token found it (A): S^T k = g A^T k and o = g A^T q +
// u (k . q), so one pass over a column's rows gives both sums. S is [dim][vdim] at
// cells[slot][(head * dim + d) * vdim + p].
template <int DPT, typename S>
__global__ void __launch_bounds__(512)
delta_rule_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ pre, int pre_ld,
                       int beta_offset, int decay_offset, const float* __restrict__ dt_bias,
                       const float* __restrict__ neg_rate, float unit_eps,
                       float* __restrict__ cells, int64_t cell_stride,
                       const int* __restrict__ q_start, const int* __restrict__ slots,
                       float* __restrict__ out, int heads, int key_heads, int dim, int vdim,
                       int chunks_per_head) {
    grid_dependency_sync();
    extern __shared__ float sm[];
    constexpr int DP = DPT * SS_SLICES;
    const int cols = (blockDim.x >> 5) * 4;
    float* q_s = sm;                          // [SS_TILE][DP]
    float* k_s = q_s + SS_TILE * DP;          // [SS_TILE][DP]
    float* v_s = k_s + SS_TILE * DP;          // [SS_TILE][cols]
    float* beta_s = v_s + SS_TILE * cols;     // [SS_TILE]
    float* kq_s = beta_s + SS_TILE;           // [SS_TILE]
    __shared__ S g_s[SS_TILE];
    const int head = blockIdx.x / chunks_per_head, chunk = blockIdx.x - head * chunks_per_head;
    const int seq = blockIdx.y;
    const int begin = q_start[seq], end = q_start[seq + 1];
    if (begin >= end) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    const int slice = lane & 7, p_local = warp * 4 + (lane >> 3);
    const int p = chunk * cols + p_local;
    const bool live = p < vdim;
    const int qk = key_heads * dim, inner = heads * vdim, width = 2 * qk + inner;
    const int kh = head / (heads / key_heads);
    float* mine = cells + (int64_t)slots[seq] * cell_stride + (int64_t)head * dim * vdim;
    S s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = slice + SS_SLICES * i;
        s[i] = (live && d < dim) ? (S)mine[(int64_t)d * vdim + p] : (S)0;
    }
    const float rate = neg_rate[head], bias = dt_bias[head];
    const float q_scale = 1.f / sqrtf((float)dim);
    for (int t0 = begin; t0 < end; t0 += SS_TILE) {
        const int nt = min(SS_TILE, end - t0);
        __syncthreads();
        for (int idx = tid; idx < nt * DP; idx += blockDim.x) {
            const int tt = idx / DP, d = idx - tt * DP;
            const float* row = qkv + (int64_t)(t0 + tt) * width + kh * dim;
            q_s[idx] = d < dim ? row[d] : 0.f;
            k_s[idx] = d < dim ? row[qk + d] : 0.f;
        }
        for (int idx = tid; idx < nt * cols; idx += blockDim.x) {
            const int tt = idx / cols, pl = idx - tt * cols;
            const int pp = chunk * cols + pl;
            v_s[idx] = pp < vdim ? qkv[(int64_t)(t0 + tt) * width + 2 * qk + head * vdim + pp] : 0.f;
        }
        if (tid < nt) {
            const float* row = pre + (int64_t)(t0 + tid) * pre_ld;
            beta_s[tid] = 1.f / (1.f + expf(-row[beta_offset + head]));
            g_s[tid] = (S)exp((double)rate * softplus_f((double)row[decay_offset + head] + (double)bias));
        }
        __syncthreads();
        // unit vectors, and the token's k . q
        for (int tt = warp; tt < nt; tt += warps) {
            float qq = 0.f, kk = 0.f, cross = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float a = q_s[tt * DP + d], b = k_s[tt * DP + d];
                qq = fmaf(a, a, qq);
                kk = fmaf(b, b, kk);
                cross = fmaf(a, b, cross);
            }
            qq = warp_sum(qq);
            kk = warp_sum(kk);
            cross = warp_sum(cross);
            const float rq = q_scale / sqrtf(qq + unit_eps), rk = 1.f / sqrtf(kk + unit_eps);
            for (int d = lane; d < dim; d += 32) {
                q_s[tt * DP + d] *= rq;
                k_s[tt * DP + d] *= rk;
            }
            if (lane == 0) kq_s[tt] = cross * rq * rk;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float* qt = q_s + tt * DP + slice;
            const float* kt = k_s + tt * DP + slice;
            S a = (S)0, b = (S)0;
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                a = fma(s[i], (S)kt[SS_SLICES * i], a);
                b = fma(s[i], (S)qt[SS_SLICES * i], b);
            }
            a = slice_sum(a);
            b = slice_sum(b);
            const S g = g_s[tt];
            const S u = (S)beta_s[tt] * ((S)v_s[tt * cols + p_local] - g * a);
#pragma unroll
            for (int i = 0; i < DPT; ++i) s[i] = fma(g, s[i], (S)kt[SS_SLICES * i] * u);
            if (slice == 0 && live)
                out[(int64_t)(t0 + tt) * inner + head * vdim + p] = (float)fma(u, (S)kq_s[tt], g * b);
        }
    }
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = slice + SS_SLICES * i;
        if (live && d < dim) mine[(int64_t)d * vdim + p] = (float)s[i];
    }
}

// ---- gated group norm ------------------------------------------------------------------------
// y: [tokens][width] float32 in `groups` equal parts; gate = silu(pre[:, gate_offset + c]).
// gate_first: out = rmsnorm_part(y * gate) * w;  else: out = rmsnorm_part(y) * w * gate.
// w has `wn` entries and is read at c % wn (one weight per feature, or one per feature of a
// part, shared by the parts). A warp per (token, part).
template <typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ pre,
                                        int pre_ld, int gate_offset, const float* __restrict__ w,
                                        int wn, int groups, int size, float eps, int gate_first,
                                        TO* __restrict__ out, int tokens) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int64_t id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (id >= (int64_t)tokens * groups) return;
    const int t = (int)(id / groups), part = (int)(id - (int64_t)t * groups);
    const int width = groups * size;
    const float* yr = y + (int64_t)t * width + part * size;
    const float* gr = pre + (int64_t)t * pre_ld + gate_offset + part * size;
    float ss = 0.f;
    for (int c = lane; c < size; c += 32) {
        float x = yr[c];
        if (gate_first) x *= silu_f(gr[c]);
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)size + eps);
    TO* orow = out + (int64_t)t * width + part * size;
    for (int c = lane; c < size; c += 32) {
        const float gate = silu_f(gr[c]);
        float x = yr[c];
        if (gate_first) x *= gate;
        x = x * rstd * w[(part * size + c) % wn];
        if (!gate_first) x *= gate;
        orow[c] = from_float<TO>(x);
    }
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_conv_act(const float* pre, int ld, int offset, const float* w, const float* bias,
                          const float* tail, long long tail_stride, const int* q_start,
                          const int* slots, const int* seq_of_token, float* out, int tokens,
                          int channels, int taps, int act, void* stream) {
    if (tokens <= 0 || channels <= 0) return MB_OK;
    if (taps < 1 || taps > 16 || tokens > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid((channels + 127) / 128, tokens);
    MB_LAUNCH((conv_act_kernel), grid, 128, 0, (cudaStream_t)stream, pre, ld, offset, w, bias, tail,
              (int64_t)tail_stride, q_start, slots, seq_of_token, out, channels, taps, act);
    return launch_status();
}

MB_EXPORT int mb_conv_tail_update(const float* pre, int ld, int offset, float* tail,
                                  long long tail_stride, const int* q_start, const int* slots,
                                  int num_seqs, int channels, int taps, void* stream) {
    if (num_seqs <= 0 || channels <= 0 || taps <= 1) return MB_OK;
    if (taps > 16 || num_seqs > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid((channels + 127) / 128, num_seqs);
    MB_LAUNCH((conv_tail_update_kernel), grid, 128, 0, (cudaStream_t)stream, pre, ld, offset, tail,
              (int64_t)tail_stride, q_start, slots, channels, taps);
    return launch_status();
}

// Warps of a scan block (each holds four columns) and the blocks a head is cut into.
static void scan_shape(int vdim, int* warps, int* chunks) {
    int w = (vdim + 3) / 4;
    if (w > 16) w = 16;
    *warps = w;
    *chunks = (vdim + 4 * w - 1) / (4 * w);
}

MB_EXPORT int mb_mamba2_scan(const float* xbc, const float* pre, int pre_ld, int dt_offset,
                             const float* dt_bias, const float* neg_rate, const float* skip,
                             float* cells, long long cell_stride, const int* q_start,
                             const int* slots, float* y, int num_seqs, int heads, int vdim,
                             int n_state, int groups, int precise, void* stream) {
    if (num_seqs <= 0) return MB_OK;
    if (heads <= 0 || vdim <= 0 || n_state <= 0 || n_state > 256 || groups <= 0 || heads % groups ||
        num_seqs > 65535)
        return MB_ERR_UNSUPPORTED_SIZE;
    int warps, chunks;
    scan_shape(vdim, &warps, &chunks);
    dim3 grid(heads * chunks, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define MB_M2_CASE(NPT)                                                                            \
    do {                                                                                           \
        const size_t smem = (size_t)(2 * SS_TILE * NPT * SS_SLICES + SS_TILE * warps * 4) *        \
                            sizeof(float);                                                         \
        if (precise)                                                                               \
            MB_LAUNCH((mamba2_scan_kernel<NPT, double>), grid, warps * 32, smem, s, xbc, pre, pre_ld,  \
                      dt_offset, dt_bias, neg_rate, skip, cells, (int64_t)cell_stride, q_start,    \
                      slots, y, heads, vdim, n_state, groups, chunks);                             \
        else                                                                                       \
            MB_LAUNCH((mamba2_scan_kernel<NPT, float>), grid, warps * 32, smem, s, xbc, pre, pre_ld,   \
                      dt_offset, dt_bias, neg_rate, skip, cells, (int64_t)cell_stride, q_start,    \
                      slots, y, heads, vdim, n_state, groups, chunks);                             \
    } while (0)
    if (n_state <= 16) MB_M2_CASE(2);
    else if (n_state <= 32) MB_M2_CASE(4);
    else if (n_state <= 64) MB_M2_CASE(8);
    else if (n_state <= 128) MB_M2_CASE(16);
    else MB_M2_CASE(32);
#undef MB_M2_CASE
    return launch_status();
}

MB_EXPORT int mb_delta_rule_scan(const float* qkv, const float* pre, int pre_ld, int beta_offset,
                                 int decay_offset, const float* dt_bias, const float* neg_rate,
                                 float unit_eps, float* cells, long long cell_stride,
                                 const int* q_start, const int* slots, float* out, int num_seqs,
                                 int heads, int key_heads, int dim, int vdim, int precise,
                                 void* stream) {
    if (num_seqs <= 0) return MB_OK;
    if (heads <= 0 || key_heads <= 0 || heads % key_heads || dim <= 0 || dim > 256 || vdim <= 0 ||
        num_seqs > 65535)
        return MB_ERR_UNSUPPORTED_SIZE;
    int warps, chunks;
    scan_shape(vdim, &warps, &chunks);
    dim3 grid(heads * chunks, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define MB_DR_CASE(DPT)                                                                            \
    do {                                                                                           \
        const size_t smem = (size_t)(2 * SS_TILE * DPT * SS_SLICES + SS_TILE * warps * 4 +         \
                                     2 * SS_TILE) * sizeof(float);                                 \
        if (precise)                                                                               \
            MB_LAUNCH((delta_rule_scan_kernel<DPT, double>), grid, warps * 32, smem, s, qkv, pre,  \
                      pre_ld, beta_offset, decay_offset, dt_bias, neg_rate, unit_eps, cells,       \
                      (int64_t)cell_stride, q_start, slots, out, heads, key_heads, dim, vdim,      \
                      chunks);                                                                     \
        else                                                                                       \
            MB_LAUNCH((delta_rule_scan_kernel<DPT, float>), grid, warps * 32, smem, s, qkv, pre,   \
                      pre_ld, beta_offset, decay_offset, dt_bias, neg_rate, unit_eps, cells,       \
                      (int64_t)cell_stride, q_start, slots, out, heads, key_heads, dim, vdim,      \
                      chunks);                                                                     \
    } while (0)
    if (dim <= 16) MB_DR_CASE(2);
    else if (dim <= 32) MB_DR_CASE(4);
    else if (dim <= 64) MB_DR_CASE(8);
    else if (dim <= 128) MB_DR_CASE(16);
    else MB_DR_CASE(32);
#undef MB_DR_CASE
    return launch_status();
}

// out_dtype: MB_F32 or MB_BF16.
MB_EXPORT int mb_gated_group_norm(const float* y, const float* pre, int pre_ld, int gate_offset,
                                  const float* w, int wn, int groups, int size, float eps,
                                  int gate_first, void* out, int out_dtype, int tokens,
                                  void* stream) {
    if (tokens <= 0) return MB_OK;
    if (groups <= 0 || size <= 0 || wn <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    const long long warps = (long long)tokens * groups;
    const long long blocks = (warps + 7) / 8;
    if (blocks > 0x7fffffffLL) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == MB_F32)
        MB_LAUNCH((gated_group_norm_kernel<float>), (int)blocks, 256, 0, s, y, pre, pre_ld, gate_offset,
                  w, wn, groups, size, eps, gate_first, (float*)out, tokens);
    else if (out_dtype == MB_BF16)
        MB_LAUNCH((gated_group_norm_kernel<__nv_bfloat16>), (int)blocks, 256, 0, s, y, pre, pre_ld,
                  gate_offset, w, wn, groups, size, eps, gate_first, (__nv_bfloat16*)out, tokens);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

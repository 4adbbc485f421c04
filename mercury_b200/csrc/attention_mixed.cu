// Attention whose heads mix their softmax weights, over the paged cache, with key heads of
// size d and value heads of size vd; and the kernel that rotates, blends and stores a
// step's keys and values for it.
//
//   w_g(i, j)  = softmax_j(q_g(i) . k(j) * scale)          over the keys j that i may see
//   w'_h(i, j) = sum_g M[h, g] w_g(i, j)                   (M: [heads, heads], may be absent)
//   o_h(i)     = sum_j w'_h(i, j) v_{kv(h)}(j)
//
// The mixed weights need the finished softmax of every head, so a block (a tile of query
// tokens with ALL their heads) walks the keys twice: once for each row's maximum and sum,
// once more to normalise, mix across heads and meet the values. Scores, weights and sums
// are float32 throughout, in both engines; the storage type T is float or bfloat16. Keys
// are walked in tiles of 32 aligned to absolute positions, so a row's arithmetic does not
// depend on how the batch was cut. Rows of a block: r = head * bq + (token in tile), at
// most 64, warp w owning the rows r = w, w + 8, ...
#include "common.cuh"

namespace mb {

constexpr int MH_WARPS = 8;
constexpr int MH_RPW = 8;                      // rows per warp
constexpr int MH_ROWS = MH_WARPS * MH_RPW;     // rows per block
constexpr int MH_KEYS = 32;

struct MixedAttentionArgs {
    const void* qkv;
    int row_width;          // elements per packed row: n_q * d + n_kv * d + n_kv * vd
    const void* k_pages;
    const void* v_pages;
    const int* table;
    int max_pages;
    const int* q_start;
    const int* kv_len;
    const float* mix;       // [n_q][n_q] or null
    void* out;              // [tokens][n_q * vd]
    int n_q, n_kv, d, vd, page_size;
    float scale;
    int window, tiles_per_seq, bq;
    // The keys of a row tile may be divided over gridDim.y blocks (decode-like batches that
    // would otherwise leave most SMs idle). mode 0: one block does everything. mode 1: a
    // block leaves its range's (maximum, sum) per row in part_ml. mode 2: a block merges the
    // ranges' (maximum, sum), weighs its own range with the finished softmax and leaves its
    // share of the output in part_out, which mixed_head_sum_kernel adds up in a fixed order.
    int num_splits, mode;
    float* part_ml;         // [tokens][n_q][splits][2]
    float* part_out;        // [tokens][n_q][splits][vd]
};

template <typename T, int NC>
__global__ void __launch_bounds__(MH_WARPS * 32)
mixed_head_attention_kernel(const MixedAttentionArgs a) {
    grid_dependency_sync();
    extern __shared__ float smem[];
    const int H = a.n_q, G = a.n_kv, d = a.d, vd = a.vd, bq = a.bq;
    const int R = H / G;
    const int seq = blockIdx.x / a.tiles_per_seq;
    const int tile = blockIdx.x - seq * a.tiles_per_seq;
    const int q_begin = a.q_start[seq];
    const int q_len = a.q_start[seq + 1] - q_begin;
    const int tok0 = tile * bq;
    if (tok0 >= q_len) return;
    const int kv_len = a.kv_len[seq];
    const int first_pos = kv_len - q_len;
    const int n_tok = min(bq, q_len - tok0);
    const int rows = H * bq;
    const T* qkv = reinterpret_cast<const T*>(a.qkv);
    const T* k_pages = reinterpret_cast<const T*>(a.k_pages);
    const T* v_pages = reinterpret_cast<const T*>(a.v_pages);

    float* q_s = smem;                               // [MH_ROWS][d]
    float* k_s = q_s + MH_ROWS * d;                  // [32][d + 1]
    float* v_s = k_s + MH_KEYS * (d + 1);            // [32][NC * 32]
    float* s_s = v_s + MH_KEYS * NC * 32;            // [MH_ROWS][32] scores, then weights
    float* m_s = s_s + MH_ROWS * MH_KEYS;            // [MH_ROWS][32] mixed weights
    float* mix_s = m_s + MH_ROWS * MH_KEYS;          // [H][H], transposed: [g][h]
    int* page_s = reinterpret_cast<int*>(mix_s + (a.mix ? H * H : 0));   // [32]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int idx = tid; idx < rows * d; idx += blockDim.x) {
        const int r = idx / d, c = idx - r * d;
        const int h = r / bq, i = r - h * bq;
        float v = 0.f;
        if (i < n_tok) v = to_float(qkv[(int64_t)(q_begin + tok0 + i) * a.row_width + h * d + c]);
        q_s[idx] = v;
    }
    if (a.mix)
        for (int idx = tid; idx < H * H; idx += blockDim.x) {
            const int h = idx / H, g = idx - h * H;
            mix_s[g * H + h] = a.mix[idx];
        }

    const int p_min = first_pos + tok0, p_max = first_pos + tok0 + n_tok - 1;
    int t_lo = 0;
    if (a.window > 0 && p_min - a.window + 1 > 0) t_lo = (p_min - a.window + 1) / MH_KEYS;
    int t_hi = p_max / MH_KEYS + 1;
    if (a.num_splits > 1) {
        const int per = (t_hi - t_lo + a.num_splits - 1) / a.num_splits;
        t_lo += (int)blockIdx.y * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }

    // this warp's rows
    int row_pos[MH_RPW];
    bool row_ok[MH_RPW];
#pragma unroll
    for (int k = 0; k < MH_RPW; ++k) {
        const int r = warp + MH_WARPS * k;
        const int h = r / bq, i = r - h * bq;
        row_ok[k] = r < rows && i < n_tok;
        row_pos[k] = first_pos + tok0 + i;
    }
    float row_m[MH_RPW], row_l[MH_RPW];
#pragma unroll
    for (int k = 0; k < MH_RPW; ++k) {
        row_m[k] = -INFINITY;
        row_l[k] = 0.f;
    }
    float acc[MH_RPW][NC];
#pragma unroll
    for (int k = 0; k < MH_RPW; ++k)
#pragma unroll
        for (int n = 0; n < NC; ++n) acc[k][n] = 0.f;

    if (a.mode == 2) {
        // the finished maximum and sum of each row, from every range's share
#pragma unroll
        for (int k = 0; k < MH_RPW; ++k) {
            if (!row_ok[k]) continue;
            const int r = warp + MH_WARPS * k;
            const int h = r / bq, i = r - h * bq;
            const float* ml = a.part_ml + ((int64_t)(q_begin + tok0 + i) * H + h) * a.num_splits * 2;
            float big = -INFINITY;
            for (int z = 0; z < a.num_splits; ++z) big = fmaxf(big, ml[2 * z]);
            float sum = 0.f;
            for (int z = 0; z < a.num_splits; ++z)
                if (ml[2 * z] > -INFINITY) sum += ml[2 * z + 1] * expf(ml[2 * z] - big);
            row_m[k] = big;
            row_l[k] = sum;
        }
    }
    const int pass_begin = a.mode == 2 ? 1 : 0, pass_end = a.mode == 1 ? 1 : 2;
    for (int pass = pass_begin; pass < pass_end; ++pass) {
        if (pass == 1) {
#pragma unroll
            for (int k = 0; k < MH_RPW; ++k) row_l[k] = row_l[k] > 0.f ? 1.f / row_l[k] : 0.f;
        }
        for (int kt = t_lo; kt < t_hi; ++kt) {
            __syncthreads();   // the tile before is consumed (and q_s, mix_s are complete)
            if (tid < MH_KEYS) {
                const int key = kt * MH_KEYS + tid;
                int page = -1;
                if (key < kv_len) page = table_page(a.table, seq, a.max_pages, key / a.page_size);
                page_s[tid] = page;
            }
            __syncthreads();
            // scores of every head against this tile's keys, one key/value head at a time
            for (int c = 0; c < G; ++c) {
                if (c > 0) __syncthreads();       // k_s is read by the scores of head c - 1
                for (int idx = tid; idx < MH_KEYS * d; idx += blockDim.x) {
                    const int j = idx / d, f = idx - j * d;
                    const int page = page_s[j];
                    float kv = 0.f;
                    if (page >= 0) {
                        const int key = kt * MH_KEYS + j;
                        kv = to_float(k_pages[(((int64_t)page * G + c) * a.page_size +
                                               (key % a.page_size)) * d + f]);
                    }
                    k_s[j * (d + 1) + f] = kv;
                }
                __syncthreads();
                const int lo = c * R * bq, hi = lo + R * bq;
                int r = lo + (((warp - lo) % MH_WARPS) + MH_WARPS) % MH_WARPS;
                const float* krow = k_s + lane * (d + 1);
                for (; r < hi; r += 4 * MH_WARPS) {
                    const float* q0 = q_s + min(r, hi - 1) * d;
                    const float* q1 = q_s + min(r + MH_WARPS, hi - 1) * d;
                    const float* q2 = q_s + min(r + 2 * MH_WARPS, hi - 1) * d;
                    const float* q3 = q_s + min(r + 3 * MH_WARPS, hi - 1) * d;
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
                    for (int f = 0; f < d; ++f) {
                        const float kv = krow[f];
                        s0 = fmaf(q0[f], kv, s0);
                        s1 = fmaf(q1[f], kv, s1);
                        s2 = fmaf(q2[f], kv, s2);
                        s3 = fmaf(q3[f], kv, s3);
                    }
                    s_s[r * MH_KEYS + lane] = s0;
                    if (r + MH_WARPS < hi) s_s[(r + MH_WARPS) * MH_KEYS + lane] = s1;
                    if (r + 2 * MH_WARPS < hi) s_s[(r + 2 * MH_WARPS) * MH_KEYS + lane] = s2;
                    if (r + 3 * MH_WARPS < hi) s_s[(r + 3 * MH_WARPS) * MH_KEYS + lane] = s3;
                }
            }
            __syncthreads();
            const int key = kt * MH_KEYS + lane;
            const bool key_ok = page_s[lane] >= 0;
            if (pass == 0) {
#pragma unroll
                for (int k = 0; k < MH_RPW; ++k) {
                    const int r = warp + MH_WARPS * k;
                    if (r >= rows) continue;
                    bool seen = row_ok[k] && key_ok && key <= row_pos[k];
                    if (a.window > 0) seen = seen && key > row_pos[k] - a.window;
                    const float sc = seen ? s_s[r * MH_KEYS + lane] * a.scale : -INFINITY;
                    const float m_new = fmaxf(row_m[k], warp_max(sc));
                    float p = 0.f, corr = 1.f;
                    if (m_new > -INFINITY) {
                        p = seen ? expf(sc - m_new) : 0.f;
                        corr = expf(row_m[k] - m_new);
                    }
                    row_l[k] = row_l[k] * corr + warp_sum(p);
                    row_m[k] = m_new;
                }
                continue;
            }
            // pass 1: finished weights of this tile, in place
#pragma unroll
            for (int k = 0; k < MH_RPW; ++k) {
                const int r = warp + MH_WARPS * k;
                if (r >= rows) continue;
                bool seen = row_ok[k] && key_ok && key <= row_pos[k];
                if (a.window > 0) seen = seen && key > row_pos[k] - a.window;
                float p = 0.f;
                if (seen) p = expf(s_s[r * MH_KEYS + lane] * a.scale - row_m[k]) * row_l[k];
                s_s[r * MH_KEYS + lane] = p;
            }
            const float* w_s = s_s;
            if (a.mix) {
                __syncthreads();
                // mixed[h][i][j] = sum_g M[h][g] w[g][i][j], four heads per thread
                const int quads = (H + 3) / 4;
                for (int item = tid; item < quads * bq * MH_KEYS; item += blockDim.x) {
                    const int j = item & 31;
                    const int i = (item >> 5) % bq;
                    const int h0 = ((item >> 5) / bq) * 4;
                    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
                    const bool b1 = h0 + 1 < H, b2 = h0 + 2 < H, b3 = h0 + 3 < H;
                    for (int g = 0; g < H; ++g) {
                        const float w = s_s[(g * bq + i) * MH_KEYS + j];
                        const float* mrow = mix_s + g * H + h0;
                        o0 = fmaf(mrow[0], w, o0);
                        if (b1) o1 = fmaf(mrow[1], w, o1);
                        if (b2) o2 = fmaf(mrow[2], w, o2);
                        if (b3) o3 = fmaf(mrow[3], w, o3);
                    }
                    m_s[(h0 * bq + i) * MH_KEYS + j] = o0;
                    if (b1) m_s[((h0 + 1) * bq + i) * MH_KEYS + j] = o1;
                    if (b2) m_s[((h0 + 2) * bq + i) * MH_KEYS + j] = o2;
                    if (b3) m_s[((h0 + 3) * bq + i) * MH_KEYS + j] = o3;
                }
                w_s = m_s;
            }
            // the values, one key/value head at a time
            for (int c = 0; c < G; ++c) {
                __syncthreads();   // weights complete / v_s consumed
                for (int idx = tid; idx < MH_KEYS * NC * 32; idx += blockDim.x) {
                    const int j = idx / (NC * 32), f = idx - j * (NC * 32);
                    const int page = page_s[j];
                    float vv = 0.f;
                    if (page >= 0 && f < vd) {
                        const int key2 = kt * MH_KEYS + j;
                        vv = to_float(v_pages[(((int64_t)page * G + c) * a.page_size +
                                               (key2 % a.page_size)) * vd + f]);
                    }
                    v_s[idx] = vv;
                }
                __syncthreads();
                bool mine[MH_RPW];
                bool any = false;
#pragma unroll
                for (int k = 0; k < MH_RPW; ++k) {
                    const int r = warp + MH_WARPS * k;
                    mine[k] = row_ok[k] && (r / bq) / R == c;
                    any = any || mine[k];
                }
                if (!any) continue;
                for (int j = 0; j < MH_KEYS; ++j) {
                    float vv[NC];
#pragma unroll
                    for (int n = 0; n < NC; ++n) vv[n] = v_s[j * NC * 32 + n * 32 + lane];
#pragma unroll
                    for (int k = 0; k < MH_RPW; ++k) {
                        if (!mine[k]) continue;
                        const float p = w_s[(warp + MH_WARPS * k) * MH_KEYS + j];
#pragma unroll
                        for (int n = 0; n < NC; ++n) acc[k][n] = fmaf(p, vv[n], acc[k][n]);
                    }
                }
            }
        }
    }

    if (a.mode != 0) {
#pragma unroll
        for (int k = 0; k < MH_RPW; ++k) {
            if (!row_ok[k]) continue;
            const int r = warp + MH_WARPS * k;
            const int h = r / bq, i = r - h * bq;
            const int64_t at = ((int64_t)(q_begin + tok0 + i) * H + h) * a.num_splits + blockIdx.y;
            if (a.mode == 1) {
                if (lane == 0) {
                    a.part_ml[at * 2] = row_m[k];
                    a.part_ml[at * 2 + 1] = row_l[k];
                }
                continue;
            }
#pragma unroll
            for (int n = 0; n < NC; ++n) {
                const int f = n * 32 + lane;
                if (f < vd) a.part_out[at * vd + f] = acc[k][n];
            }
        }
        return;
    }
    T* out = reinterpret_cast<T*>(a.out);
#pragma unroll
    for (int k = 0; k < MH_RPW; ++k) {
        if (!row_ok[k]) continue;
        const int r = warp + MH_WARPS * k;
        const int h = r / bq, i = r - h * bq;
        const int64_t at = ((int64_t)(q_begin + tok0 + i) * H + h) * vd;
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            const int f = n * 32 + lane;
            if (f < vd) out[at + f] = from_float<T>(acc[k][n]);
        }
    }
}

// out[token][head][:] = sum over the ranges, in ascending order; padding tokens get zeros.
template <typename T>
__global__ void mixed_head_sum_kernel(const float* __restrict__ part_out,
                                      const int* __restrict__ seq_of_token, T* __restrict__ out,
                                      int n_q, int vd, int num_splits) {
    grid_dependency_sync();
    const int tok = blockIdx.x, head = blockIdx.y;
    const int64_t flat = (int64_t)tok * n_q + head;
    const bool live = seq_of_token[tok] >= 0;
    for (int f = threadIdx.x; f < vd; f += blockDim.x) {
        float v = 0.f;
        if (live)
            for (int z = 0; z < num_splits; ++z) v += part_out[(flat * num_splits + z) * vd + f];
        out[flat * vd + f] = from_float<T>(v);
    }
}

int launch_mixed_head_sum(const float* part_out, const int* seq_of_token, void* out, int tokens,
                          int n_q, int vd, int num_splits, int dtype, cudaStream_t s) {
    dim3 grid(tokens, n_q);
    if (dtype == MB_F32)
        MB_LAUNCH((mixed_head_sum_kernel<float>), grid, 64, 0, s, part_out, seq_of_token, (float*)out,
                  n_q, vd, num_splits);
    else
        MB_LAUNCH((mixed_head_sum_kernel<__nv_bfloat16>), grid, 64, 0, s, part_out, seq_of_token,
                  (__nv_bfloat16*)out, n_q, vd, num_splits);
    return launch_status();
}

template <typename T, int NC>
int launch_mixed_attention(const MixedAttentionArgs& a, int num_seqs, cudaStream_t s) {
    const size_t smem = (size_t)(MH_ROWS * a.d + MH_KEYS * (a.d + 1) + MH_KEYS * NC * 32 +
                                 2 * MH_ROWS * MH_KEYS + (a.mix ? a.n_q * a.n_q : 0)) * sizeof(float) +
                        MH_KEYS * sizeof(int);
    static size_t raised = 0;   // per instantiation
    if (smem > 48 * 1024 && smem > raised) {
        if (cudaFuncSetAttribute(mixed_head_attention_kernel<T, NC>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = smem;
    }
    dim3 grid(num_seqs * a.tiles_per_seq, a.num_splits);
    MB_LAUNCH((mixed_head_attention_kernel<T, NC>), grid, MH_WARPS * 32, smem, s, a);
    return launch_status();
}

template <typename T>
int dispatch_mixed_attention(const MixedAttentionArgs& a, int num_seqs, cudaStream_t s) {
    switch ((a.vd + 31) / 32) {
        case 1: return launch_mixed_attention<T, 1>(a, num_seqs, s);
        case 2: return launch_mixed_attention<T, 2>(a, num_seqs, s);
        case 3: return launch_mixed_attention<T, 3>(a, num_seqs, s);
        case 4: return launch_mixed_attention<T, 4>(a, num_seqs, s);
        case 5: return launch_mixed_attention<T, 5>(a, num_seqs, s);
        case 6: return launch_mixed_attention<T, 6>(a, num_seqs, s);
        case 7: return launch_mixed_attention<T, 7>(a, num_seqs, s);
        case 8: return launch_mixed_attention<T, 8>(a, num_seqs, s);
    }
    return MB_ERR_UNSUPPORTED_SIZE;
}

// ------------------------------------------------------------------ rotate, blend, store
// One block per token of a packed row [n_q heads of d | n_kv heads of d | n_kv heads of vd].
// q and k: the first `rot` features of each head are rotated in place (feature i with
// i + rot/2, by the float32 tables cos/sin [positions][rot/2]); the rest pass unchanged.
// v: copied to `keep` (if given), then blended with `blend_from` (if given):
// v <- (1 - c) v + c blend_from, c = *blend. Rotated keys and blended values go into the
// token's slot of the pages. Tokens of sequence -1 are padding; a page of -1 is never written.
template <typename T>
__global__ void rope_blend_store_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, int rot,
                                        const int* __restrict__ positions,
                                        const int* __restrict__ seq_of_token,
                                        const int* __restrict__ table, int max_pages,
                                        T* __restrict__ k_pages, T* __restrict__ v_pages,
                                        const T* __restrict__ blend_from,
                                        const float* __restrict__ blend, T* __restrict__ keep,
                                        int n_q, int n_kv, int d, int vd, int page_size, int store) {
    grid_dependency_sync();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int pos = checked_position(positions[t]);
    const int half = rot / 2;
    const int width = (n_q + n_kv) * d + n_kv * vd;
    T* row = qkv + (int64_t)t * width;
    int64_t slot = -1;
    if (store) {
        const int page = table_page(table, seq, max_pages, pos / page_size);
        if (page >= 0) slot = (int64_t)page * n_kv * page_size + pos % page_size;
    }
    const int per_head = d - half;
    for (int w = threadIdx.x; w < (n_q + n_kv) * per_head; w += blockDim.x) {
        const int head = w / per_head;
        const int i = w - head * per_head;
        T* x = row + (int64_t)head * d;
        T* dst = nullptr;
        if (head >= n_q && slot >= 0) dst = k_pages + (slot + (int64_t)(head - n_q) * page_size) * d;
        if (i < half) {
            const float a = to_float(x[i]), b = to_float(x[i + half]);
            const float c = cos_t[(int64_t)pos * half + i], s = sin_t[(int64_t)pos * half + i];
            const T ta = from_float<T>(a * c - b * s), tb = from_float<T>(b * c + a * s);
            x[i] = ta;
            x[i + half] = tb;
            if (dst) {
                dst[i] = ta;
                dst[i + half] = tb;
            }
        } else if (dst) {
            dst[i + half] = x[i + half];
        }
    }
    T* v = row + (int64_t)(n_q + n_kv) * d;
    const int v_size = n_kv * vd;
    const float c = blend_from ? *blend : 0.f;
    for (int w = threadIdx.x; w < v_size; w += blockDim.x) {
        T val = v[w];
        if (keep) keep[(int64_t)t * v_size + w] = val;
        if (blend_from) {
            val = from_float<T>((1.f - c) * to_float(val) + c * to_float(blend_from[(int64_t)t * v_size + w]));
            v[w] = val;
        }
        if (slot >= 0) {
            const int head = w / vd, i = w - head * vd;
            v_pages[(slot + (int64_t)head * page_size) * vd + i] = val;
        }
    }
}

}  // namespace mb

using namespace mb;

// Floats of scratch that `num_splits` ranges need for `tokens` rows of the batch.
MB_EXPORT long long mb_mixed_head_scratch_floats(int tokens, int n_q, int vd, int num_splits) {
    return num_splits <= 1 ? 0 : (long long)tokens * n_q * num_splits * (vd + 2);
}

MB_EXPORT int mb_mixed_head_attention(const void* qkv, int row_width, const void* k_pages,
                                      const void* v_pages, const int* table, int max_pages,
                                      const int* q_start, const int* kv_len, const float* mix,
                                      void* out, int num_seqs, int max_q_len, int n_q, int n_kv,
                                      int d, int vd, int page_size, float scale, int window,
                                      int dtype, int num_splits, const int* seq_of_token,
                                      int tokens, float* scratch, long long scratch_floats,
                                      void* stream) {
    if (num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (d <= 0 || d > 256 || vd <= 0 || vd > 256 || n_kv <= 0 || n_q % n_kv || n_q > MH_ROWS)
        return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || (page_size & (page_size - 1))) return MB_ERR_UNSUPPORTED_SIZE;
    MixedAttentionArgs a;
    a.qkv = qkv; a.row_width = row_width; a.k_pages = k_pages; a.v_pages = v_pages;
    a.table = table; a.max_pages = max_pages; a.q_start = q_start; a.kv_len = kv_len;
    a.mix = mix; a.out = out; a.n_q = n_q; a.n_kv = n_kv; a.d = d; a.vd = vd;
    a.page_size = page_size; a.scale = scale; a.window = window;
    int bq = MH_ROWS / n_q;
    if (bq > 16) bq = 16;
    if (bq > max_q_len) bq = max_q_len;
    a.bq = bq;
    a.tiles_per_seq = (max_q_len + bq - 1) / bq;
    a.num_splits = 1;
    a.mode = 0;
    a.part_ml = a.part_out = nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype != MB_F32 && dtype != MB_BF16) return MB_ERR_BAD_DTYPE;
    if (num_splits <= 1)
        return dtype == MB_F32 ? dispatch_mixed_attention<float>(a, num_seqs, s)
                               : dispatch_mixed_attention<__nv_bfloat16>(a, num_seqs, s);
    if (num_splits > 65535 || n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (!scratch || scratch_floats < mb_mixed_head_scratch_floats(tokens, n_q, vd, num_splits))
        return MB_ERR_SCRATCH;
    a.num_splits = num_splits;
    a.part_out = scratch;
    a.part_ml = scratch + (int64_t)tokens * n_q * num_splits * vd;
    for (int mode = 1; mode <= 2; ++mode) {
        a.mode = mode;
        const int rc = dtype == MB_F32 ? dispatch_mixed_attention<float>(a, num_seqs, s)
                                       : dispatch_mixed_attention<__nv_bfloat16>(a, num_seqs, s);
        if (rc != MB_OK) return rc;
    }
    return launch_mixed_head_sum(a.part_out, seq_of_token, out, tokens, n_q, vd, num_splits, dtype, s);
}

MB_EXPORT int mb_rope_blend_store(void* qkv, const float* cos_t, const float* sin_t, int rot,
                                  const int* positions, const int* seq_of_token, const int* table,
                                  int max_pages, void* k_pages, void* v_pages,
                                  const void* blend_from, const float* blend, void* keep, int tokens,
                                  int n_q, int n_kv, int d, int vd, int page_size, int store,
                                  int dtype, void* stream) {
    if (tokens <= 0) return MB_OK;
    if (rot < 0 || rot > d || (rot & 1) || (rot && !cos_t)) return MB_ERR_UNSUPPORTED_SIZE;
    if (blend_from && !blend) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    if (dtype == MB_F32)
        MB_LAUNCH((rope_blend_store_kernel<float>), tokens, 256, 0, s, (float*)qkv, cos_t, sin_t, rot,
                  positions, seq_of_token, table, max_pages, (float*)k_pages, (float*)v_pages,
                  (const float*)blend_from, blend, (float*)keep, n_q, n_kv, d, vd, page_size, store);
    else if (dtype == MB_BF16)
        MB_LAUNCH((rope_blend_store_kernel<bf>), tokens, 256, 0, s, (bf*)qkv, cos_t, sin_t, rot,
                  positions, seq_of_token, table, max_pages, (bf*)k_pages, (bf*)v_pages,
                  (const bf*)blend_from, blend, (bf*)keep, n_q, n_kv, d, vd, page_size, store);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}
